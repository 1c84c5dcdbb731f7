// Attention whose keys and values have sizes of their own, over a paged cache, with rotated queries and keys.
//
// The cache of one layer is K [block][kv_head][BT][dk] and V [block][kv_head][BT][dv] (dk: the size of queries and
// keys, dv: of values; they need not be equal).  Query head h reads key/value head h / (H / Hkv).  A window w > 0
// hides keys at or before position − w; w = 0 is plain causal attention.
//
// qkv_rope_append: the float32 result of a layer's input product holds, per token, the queries (H·dk columns at
//   q_off), keys (Hkv·dk at k_off) and values (Hkv·dv at v_off), biases included.  Of every query and key head the
//   first `rot` entries are rotated by the token's position: entry i pairs with entry i + rot/2, and the pair (a, b)
//   becomes (a cos t − b sin t, b cos t + a sin t) with t = position · freq[i] (float32; freq holds whatever scaling
//   of the frequencies the model asks for).  Queries go to a matrix of their own in the activation dtype, keys and
//   values into the cache at (slot, position).
// attn_window: one warp per (token, head) walks the visible keys of the token's slot in chunks of 32 with an online
//   softmax in float32; any mix of prompt tokens and single tokens.  Every size (dk, dv ≤ 256) is taken; the 32-bit
//   path's attention, and the fallback of the bfloat16 path.  The result is multiplied by out_scale (a mixer that
//   sums several branches puts a branch's weight there) and written at a column offset of wider rows.
#include "common.cuh"

namespace {
constexpr int AW_WARPS = 4;
constexpr int AW_MAX = 256;

template <typename ET>
__global__ void __launch_bounds__(128)
qkv_rope_append_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ freq,
                       int rot, ET* __restrict__ q_out, int ldq, ET* __restrict__ Kc, ET* __restrict__ Vc,
                       const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                       const int* __restrict__ tok_pos, int H, int Hkv, int dk, int dv, int BT, int write_cache,
                       int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;  // padding row (the whole CTA leaves: no barrier is missed)
    const int pos = tok_pos[t];
    const float* row = proj + (size_t)t * ld;
    const int half = rot / 2;
    // the token's cosines and sines once, for all heads: [half] each
    extern __shared__ float cs_sm[];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * freq[i], &cs_sm[half + i], &cs_sm[i]);
    __syncthreads();
    auto rotated = [&](const float* head, int c) -> float {
        if (c >= rot) return head[c];
        if (c < half) return head[c] * cs_sm[c] - head[c + half] * cs_sm[half + c];
        return head[c] * cs_sm[c - half] + head[c - half] * cs_sm[c];
    };
    for (int i = threadIdx.x; i < H * dk; i += blockDim.x) {
        const int h = i / dk, c = i - h * dk;
        ElemIO<ET>::store(q_out + (size_t)t * ldq + i, rotated(row + q_off + h * dk, c));
    }
    if (!write_cache) return;
    const int bi = pos / BT;
    const int blk = (pos >= 0 && bi < max_blocks) ? block_table[(size_t)slot * max_blocks + bi] : -1;
    if (blk < 0) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        return;
    }
    for (int i = threadIdx.x; i < Hkv * dk; i += blockDim.x) {
        const int h = i / dk, c = i - h * dk;
        ElemIO<ET>::store(Kc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dk + c, rotated(row + k_off + h * dk, c));
    }
    for (int i = threadIdx.x; i < Hkv * dv; i += blockDim.x) {
        const int h = i / dv, c = i - h * dv;
        ElemIO<ET>::store(Vc + (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dv + c, row[v_off + i]);
    }
}

template <typename ET>
__global__ void __launch_bounds__(AW_WARPS * 32)
attn_window_kernel(const ET* __restrict__ q_in, int ldq, const ET* __restrict__ Kc, const ET* __restrict__ Vc,
                   const int* __restrict__ block_table, int max_blocks, const int* __restrict__ tok_slot,
                   const int* __restrict__ tok_pos, ET* __restrict__ out, int ld_out, int H, int Hkv, int dk, int dv, int BT,
                   float scale, int window, float out_scale, int* __restrict__ dev_err) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float q_sm[];  // [AW_WARPS][dk]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * AW_WARPS + warp;
    const int slot = tok_slot[t];
    if (h >= H || slot < 0) return;  // whole warp leaves together; no block-wide barrier below
    const int pos = tok_pos[t];
    const int hk = h / (H / Hkv);
    float* q = q_sm + warp * dk;
    const ET* qsrc = q_in + (size_t)t * ldq + (size_t)h * dk;
    for (int i = lane; i < dk; i += 32) q[i] = ElemIO<ET>::load(qsrc + i) * scale;
    __syncwarp();

    float acc[AW_MAX / 32];
#pragma unroll
    for (int i = 0; i < AW_MAX / 32; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)slot * max_blocks;
    bool lost = false;

    for (int k0 = (first / 32) * 32; k0 <= pos; k0 += 32) {
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const size_t kbase = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dk;
        const size_t vbase = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dv;
        const int key = k0 + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const ET* krow = Kc + kbase + (size_t)lane * dk;
            float dot = 0.f;
            for (int c = 0; c < dk; ++c) dot = fmaf(q[c], ElemIO<ET>::load(krow + c), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));      // at least one key of the chunk is valid
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < AW_MAX / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, pos - k0 + 1);
        for (int j = 0; j < n_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.f) continue;  // uniform across the warp
            const ET* vrow = Vc + vbase + (size_t)j * dv;
#pragma unroll
            for (int i = 0; i < AW_MAX / 32; ++i) {
                const int c = i * 32 + lane;
                if (c < dv) acc[i] = fmaf(pj, ElemIO<ET>::load(vrow + c), acc[i]);
            }
        }
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    const float inv = (l > 0.f) ? out_scale / l : 0.f;
    ET* dst = out + (size_t)t * ld_out + (size_t)h * dv;
#pragma unroll
    for (int i = 0; i < AW_MAX / 32; ++i) {
        const int c = i * 32 + lane;
        if (c < dv) ElemIO<ET>::store(dst + c, acc[i] * inv);
    }
}
}  // namespace

extern "C" int vlrf_qkv_rope_append(const float* proj, int ld, int q_off, int k_off, int v_off, const float* freq, int rot,
                                    void* q_out, int ldq, void* Kc, void* Vc, int dtype, const int* block_table, int max_blocks,
                                    const int* tok_slot, const int* tok_pos, int T, int H, int Hkv, int dk, int dv, int BT,
                                    int write_cache, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && Hkv > 0 && dk > 0 && dv > 0 && BT > 0 && max_blocks > 0, "qkv_rope_append: bad sizes");
    VLRF_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dk, "qkv_rope_append: %d rotated entries of a head of %d", rot, dk);
    VLRF_REQUIRE(rot == 0 || freq != nullptr, "qkv_rope_append: a rotation needs its frequencies");
    VLRF_REQUIRE(q_off + H * dk <= ld && k_off + Hkv * dk <= ld && v_off + Hkv * dv <= ld && ldq >= H * dk,
                 "qkv_rope_append: columns lie outside the row");
    VLRF_REQUIRE(dev_err != nullptr, "qkv_rope_append: needs the device error word");
    if (T == 0) return VLRF_OK;
    if (dtype == VLRF_F32)
        launch_chained(qkv_rope_append_kernel<float>, dim3(T), dim3(128), (size_t)rot * sizeof(float), stream, proj, ld, q_off, k_off, v_off, freq, rot,
                       (float*)q_out, ldq, (float*)Kc, (float*)Vc, block_table, max_blocks, tok_slot, tok_pos, H, Hkv, dk, dv, BT,
                       write_cache, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(qkv_rope_append_kernel<__nv_bfloat16>, dim3(T), dim3(128), (size_t)rot * sizeof(float), stream, proj, ld, q_off, k_off, v_off, freq,
                       rot, (__nv_bfloat16*)q_out, ldq, (__nv_bfloat16*)Kc, (__nv_bfloat16*)Vc, block_table, max_blocks, tok_slot,
                       tok_pos, H, Hkv, dk, dv, BT, write_cache, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "qkv_rope_append: unknown dtype %d", dtype);
    return vlrf_check_launch("qkv_rope_append");
}

extern "C" int vlrf_attn_window(const void* q, int dtype, int ldq, const void* Kc, const void* Vc, const int* block_table,
                                int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T, int H,
                                int Hkv, int dk, int dv, int BT, float scale, int window, float out_scale, int* dev_err,
                                cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "attn_window: bad sizes");
    VLRF_REQUIRE(H % Hkv == 0, "attn_window: %d heads cannot share %d key/value heads", H, Hkv);
    VLRF_REQUIRE(dk > 0 && dk <= AW_MAX && dv > 0 && dv <= AW_MAX, "attn_window: head sizes %d and %d are not in 1…%d", dk, dv, AW_MAX);
    VLRF_REQUIRE(BT % 32 == 0, "attn_window: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(window >= 0, "attn_window: negative window");
    VLRF_REQUIRE(ldq >= H * dk && ld_out >= H * dv, "attn_window: leading sizes are smaller than the rows");
    VLRF_REQUIRE(dev_err != nullptr, "attn_window: needs the device error word");
    if (T == 0) return VLRF_OK;
    dim3 grid(T, (H + AW_WARPS - 1) / AW_WARPS);
    const size_t smem = (size_t)AW_WARPS * dk * sizeof(float);
    if (dtype == VLRF_F32)
        launch_chained(attn_window_kernel<float>, grid, dim3(AW_WARPS * 32), smem, stream, (const float*)q, ldq, (const float*)Kc,
                       (const float*)Vc, block_table, max_blocks, tok_slot, tok_pos, (float*)out, ld_out, H, Hkv, dk, dv, BT, scale,
                       window, out_scale, dev_err);
    else if (dtype == VLRF_BF16)
        launch_chained(attn_window_kernel<__nv_bfloat16>, grid, dim3(AW_WARPS * 32), smem, stream, (const __nv_bfloat16*)q, ldq,
                       (const __nv_bfloat16*)Kc, (const __nv_bfloat16*)Vc, block_table, max_blocks, tok_slot, tok_pos,
                       (__nv_bfloat16*)out, ld_out, H, Hkv, dk, dv, BT, scale, window, out_scale, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "attn_window: unknown dtype %d", dtype);
    return vlrf_check_launch("attn_window");
}
