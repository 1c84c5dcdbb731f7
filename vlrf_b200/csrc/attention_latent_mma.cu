// Attention over a cache of latents on the tensor cores (bfloat16, `mma.sync`), for prompt steps and decode steps.
//
// What is computed is attention_latent.cu's: per head h, scores (q'_h · row_j) · scale over the visible rows j of the
// token's slot, softmax in float32, output Σ_j p_j c_j (the row's first C numbers).  All heads of a token attend the
// same rows, so the heads are the 16 rows of the MMAs: a token's 16 heads (fewer: the rest are zero rows; more: a CTA
// per group of 16) against tiles of 32 cache rows that lie in shared memory once, however many heads read them.
//
// A token group is four warps.  For a tile, warp w multiplies the 16 queries by rows 8w … 8w+7 (k = all C + R
// columns), scales, masks, and leaves its 16 × 8 scores in shared memory; after a barrier every warp reads the whole
// 16 × 32 tile of scores, keeps the running maximum and sum of its rows (the same numbers in every warp), and adds
// P · rows[:, its quarter of the C columns] to its accumulators (P rounded to bfloat16, as an MMA operand).  A CTA
// holds G such groups for G consecutive tokens of one sequence (prompt steps: the tile is fetched once for all of
// them), or one token and one part of its context (decode steps: the parts' results, unnormalised with their maximum
// and sum, meet in a second kernel).  Tiles arrive by `cp.async` into two buffers; rows behind the last visible one are
// filled with zeros, so nothing unwritten is ever multiplied.
//
// Sizes taken: C a multiple of 32 up to 512, R a multiple of 16, cache rows of a multiple of 8 numbers, blocks of a
// multiple of 32 tokens.  Others go to attention_latent.cu.
#include "common.cuh"

namespace {
constexpr int LM_KT = 32;            // cache rows a tile
constexpr int LM_NT_MAX = 16;        // 8-column tiles of the output a warp (C ≤ 4 · 16 · 8)
constexpr int LM_SPAD = 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// G: tokens (groups of four warps) a CTA.  grid (sequences · tiles of G tokens, groups of 16 heads, parts of the context)
template <int G>
__global__ void __launch_bounds__(G * 128)
attn_latent_mma_kernel(const __nv_bfloat16* __restrict__ qp, int ld_q, const __nv_bfloat16* __restrict__ cache, int row_w,
                       int C, int R, const int* __restrict__ block_table, int max_blocks, const int* __restrict__ seq_slot,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, int tiles_per_seq,
                       __nv_bfloat16* __restrict__ out, int ld_out, int H, int BT, float scale, int window, int n_split,
                       float* __restrict__ partials, int* __restrict__ dev_err) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char lm_raw[];
    const int D = C + R, ldk = D + 8;                              // shared rows padded by 16 bytes: ldmatrix without conflicts
    __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(lm_raw);                     // [G][16][ldk]
    __nv_bfloat16* k_sm = q_sm + (size_t)G * 16 * ldk;                                  // [2][LM_KT][ldk]
    float* s_sm = reinterpret_cast<float*>(k_sm + (size_t)2 * LM_KT * ldk);             // [G][2][16][LM_KT + LM_SPAD]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = warp >> 2, w = warp & 3, g = lane >> 2, t4 = lane & 3;
    const int seq = blockIdx.x / tiles_per_seq, tile_in_seq = blockIdx.x % tiles_per_seq;
    const int hg = blockIdx.y, split = blockIdx.z;
    const int slot = seq_slot[seq];
    const int row0 = seq_start[seq] + tile_in_seq * G, row_end = seq_start[seq + 1];
    if (row0 >= row_end) return;                                   // the sequence has fewer tokens than the longest
    const int n_here = min(G, row_end - row0);
    const int pos0 = seq_pos0[seq] + tile_in_seq * G;              // position of the CTA's first token
    const int heads_here = min(16, H - hg * 16);
    const int nt_cnt = C >> 5;                                     // 8-column tiles a warp
    const int cw = C >> 2;                                         // columns a warp

    if (slot < 0) {                                                // padding rows: zeros (no part writes anything)
        if (split == 0)
            for (int i = tid; i < n_here * heads_here * C; i += G * 128) {
                const int r = i / (heads_here * C), rest = i - r * heads_here * C;
                out[(size_t)(row0 + r) * ld_out + (size_t)hg * 16 * C + rest] = __float2bfloat16_rn(0.f);
            }
        return;
    }
    // the queries: 16 rows a token, rows beyond the heads are zeros
    for (int i = tid; i < G * 16 * (D >> 3); i += G * 128) {
        const int c8 = i % (D >> 3), r = (i / (D >> 3)) & 15, gi = i / ((D >> 3) * 16);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (gi < n_here && r < heads_here)
            v = *reinterpret_cast<const uint4*>(qp + (size_t)(row0 + gi) * ld_q + (size_t)(hg * 16 + r) * D + c8 * 8);
        *reinterpret_cast<uint4*>(q_sm + ((size_t)gi * 16 + r) * ldk + c8 * 8) = v;
    }
    // the tiles of this CTA: those of the last token's visible rows, this part's share of them
    const int last_pos = pos0 + n_here - 1;
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    int tile_lo = first_key / LM_KT, tile_hi = last_pos / LM_KT + 1;
    if (n_split > 1) {
        const int per = (tile_hi - tile_lo + n_split - 1) / n_split;
        tile_lo = tile_lo + split * per;
        tile_hi = min(tile_hi, tile_lo + per);
    }
    const int* table = block_table + (size_t)slot * max_blocks;
    const int chunks = D >> 3;                                     // 16-byte pieces a row
    auto fetch = [&](int tile, int buf) {
        const int key0 = tile * LM_KT;
        const int blk = table[key0 / BT];
        if (blk < 0 && tid == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        const __nv_bfloat16* src = cache + ((size_t)max(blk, 0) * BT + (key0 % BT)) * row_w;
        __nv_bfloat16* dst = k_sm + (size_t)buf * LM_KT * ldk;
        for (int i = tid; i < LM_KT * chunks; i += G * 128) {
            const int r = i / chunks, c8 = i - r * chunks;
            const bool live = blk >= 0 && key0 + r <= last_pos;    // rows nobody may see arrive as zeros
            cp_async_16(smem_u32(dst + (size_t)r * ldk + c8 * 8), src + (size_t)r * row_w + c8 * 8, live ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int my_pos = pos0 + grp;                                 // this group's token
    const bool active = grp < n_here;
    const int my_first = window > 0 ? max(0, my_pos - window + 1) : 0;
    float acc[LM_NT_MAX][4];
#pragma unroll
    for (int i = 0; i < LM_NT_MAX; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (tile_lo < tile_hi) fetch(tile_lo, 0);
    const uint32_t q_base = smem_u32(q_sm + (size_t)grp * 16 * ldk);
    float* s_grp = s_sm + (size_t)grp * 2 * 16 * (LM_KT + LM_SPAD);
    for (int tile = tile_lo; tile < tile_hi; ++tile) {
        const int buf = (tile - tile_lo) & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                           // the tile has landed; the other buffer is free
        if (tile + 1 < tile_hi) fetch(tile + 1, buf ^ 1);
        const __nv_bfloat16* kt = k_sm + (size_t)buf * LM_KT * ldk;
        const int key0 = tile * LM_KT;
        float* s_buf = s_grp + (size_t)buf * 16 * (LM_KT + LM_SPAD);
        const bool tile_live = active && key0 <= my_pos && key0 + LM_KT > my_first;
        if (tile_live) {
            // scores of the 16 heads against rows 8w … 8w+7
            // (four sums side by side: one chain of dependent MMAs over all of k would wait for each one's latency)
            float sc[4] = {0.f, 0.f, 0.f, 0.f}, sc1[4] = {0.f, 0.f, 0.f, 0.f}, sc2[4] = {0.f, 0.f, 0.f, 0.f}, sc3[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t a_addr = q_base + (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ldk + 8 * (lane >> 4)) * 2;
            const uint32_t b_addr = smem_u32(kt) + (uint32_t)((8 * w + (lane & 7)) * ldk + 8 * ((lane >> 3) & 1)) * 2;
            int kk = 0;
            for (; kk + 64 <= D; kk += 64) {
                uint32_t a0[4], a1[4], a2[4], a3[4], b[8];
                ldsm_x4(a0, a_addr + kk * 2);        ldsm_x2(b[0], b[1], b_addr + kk * 2);
                ldsm_x4(a1, a_addr + (kk + 16) * 2); ldsm_x2(b[2], b[3], b_addr + (kk + 16) * 2);
                ldsm_x4(a2, a_addr + (kk + 32) * 2); ldsm_x2(b[4], b[5], b_addr + (kk + 32) * 2);
                ldsm_x4(a3, a_addr + (kk + 48) * 2); ldsm_x2(b[6], b[7], b_addr + (kk + 48) * 2);
                mma_16816(sc, a0, b[0], b[1]);
                mma_16816(sc1, a1, b[2], b[3]);
                mma_16816(sc2, a2, b[4], b[5]);
                mma_16816(sc3, a3, b[6], b[7]);
            }
            for (; kk < D; kk += 16) {
                uint32_t a[4], b0, b1;
                ldsm_x4(a, a_addr + kk * 2);
                ldsm_x2(b0, b1, b_addr + kk * 2);
                mma_16816(sc, a, b0, b1);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[e] = (sc[e] + sc1[e]) + (sc2[e] + sc3[e]);
            const int kcol = key0 + 8 * w + 2 * t4;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = kcol + (e & 1);
                sc[e] = (key <= my_pos && key >= my_first) ? sc[e] * scale : -INFINITY;
            }
            *reinterpret_cast<float2*>(s_buf + g * (LM_KT + LM_SPAD) + 8 * w + 2 * t4) = make_float2(sc[0], sc[1]);
            *reinterpret_cast<float2*>(s_buf + (g + 8) * (LM_KT + LM_SPAD) + 8 * w + 2 * t4) = make_float2(sc[2], sc[3]);
        }
        __syncthreads();                                           // every warp's scores of the tile are there
        if (tile_live) {
            // rows g and g + 8: this thread holds keys 16kk + 2t4 (+1) and 16kk + 2t4 + 8 (+1) of each
            float s[2][2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int r = 0; r < 2; ++r)
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    const float* p = s_buf + (g + 8 * r) * (LM_KT + LM_SPAD) + 16 * kk + 2 * t4;
                    const float2 lo = *reinterpret_cast<const float2*>(p), hi = *reinterpret_cast<const float2*>(p + 8);
                    s[r][kk][0] = lo.x; s[r][kk][1] = lo.y; s[r][kk][2] = hi.x; s[r][kk][3] = hi.y;
                    mx[r] = fmaxf(mx[r], fmaxf(fmaxf(lo.x, lo.y), fmaxf(hi.x, hi.y)));
                }
            float corr[2];
            uint32_t pa[2][4];                                     // P as the A operand of two k-steps
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_run[r], mx[r]);        // the tile holds a visible key, so m_new is a number
                corr[r] = (m_run[r] == -INFINITY) ? 0.f : expf(m_run[r] - m_new);
                float sum = 0.f;
#pragma unroll
                for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // (what enters the sum is what the MMA multiplies: P rounded to bfloat16)
                        const float p = __bfloat162float(__float2bfloat16_rn(expf(s[r][kk][e] - m_new)));
                        s[r][kk][e] = p;
                        sum += p;
                    }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                l_run[r] = l_run[r] * corr[r] + sum;
                m_run[r] = m_new;
            }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                pa[kk][0] = pack_bf16(s[0][kk][0], s[0][kk][1]);   // (row g,     k 2t4, 2t4+1)
                pa[kk][1] = pack_bf16(s[1][kk][0], s[1][kk][1]);   // (row g + 8, k 2t4, 2t4+1)
                pa[kk][2] = pack_bf16(s[0][kk][2], s[0][kk][3]);   // (row g,     k 2t4+8, +9)
                pa[kk][3] = pack_bf16(s[1][kk][2], s[1][kk][3]);   // (row g + 8, k 2t4+8, +9)
            }
            const uint32_t v_addr = smem_u32(kt) + (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ldk + w * cw) * 2;
#pragma unroll
            for (int nt = 0; nt < LM_NT_MAX; ++nt) {
                if (nt < nt_cnt) { acc[nt][0] *= corr[0]; acc[nt][1] *= corr[0]; acc[nt][2] *= corr[1]; acc[nt][3] *= corr[1]; }
            }
            // four column tiles at a time: their operands are requested together, then the four MMAs follow, so that
            // one wait for shared memory covers four of them (the statements keep their order in the program)
#pragma unroll
            for (int nt0 = 0; nt0 < LM_NT_MAX; nt0 += 4) {
                if (nt0 < nt_cnt) {
#pragma unroll
                    for (int kk = 0; kk < 2; ++kk) {
                        uint32_t b[4][2];
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (nt0 + i < nt_cnt) ldsm_x2_trans(b[i][0], b[i][1], v_addr + (uint32_t)(16 * kk * ldk + (nt0 + i) * 8) * 2);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (nt0 + i < nt_cnt) mma_16816(acc[nt0 + i], pa[kk], b[i][0], b[i][1]);
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (!active) return;
    const int tok = row0 + grp;
    if (n_split == 1) {
        const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
        for (int nt = 0; nt < LM_NT_MAX; ++nt) {
            if (nt < nt_cnt) {
                const int col = w * cw + nt * 8 + 2 * t4;
                if (g < heads_here)
                    *reinterpret_cast<uint32_t*>(out + (size_t)tok * ld_out + (size_t)(hg * 16 + g) * C + col) = pack_bf16(acc[nt][0] * inv0, acc[nt][1] * inv0);
                if (g + 8 < heads_here)
                    *reinterpret_cast<uint32_t*>(out + (size_t)tok * ld_out + (size_t)(hg * 16 + g + 8) * C + col) = pack_bf16(acc[nt][2] * inv1, acc[nt][3] * inv1);
            }
        }
        return;
    }
    // a part of a context: per head the unnormalised sums, then the maximum and the sum of the weights
    float* part = partials + (((size_t)tok * gridDim.y + hg) * n_split + split) * 16 * (C + 2);
#pragma unroll
    for (int nt = 0; nt < LM_NT_MAX; ++nt) {
        if (nt < nt_cnt) {
            const int col = w * cw + nt * 8 + 2 * t4;
            *reinterpret_cast<float2*>(part + (size_t)g * (C + 2) + col) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(part + (size_t)(g + 8) * (C + 2) + col) = make_float2(acc[nt][2], acc[nt][3]);
        }
    }
    if (w == 0 && t4 == 0) {
        part[(size_t)g * (C + 2) + C] = m_run[0]; part[(size_t)g * (C + 2) + C + 1] = l_run[0];
        part[(size_t)(g + 8) * (C + 2) + C] = m_run[1]; part[(size_t)(g + 8) * (C + 2) + C + 1] = l_run[1];
    }
}

// the parts of every (token, head) into one: weights exp(m_s − max m) on the parts' unnormalised sums
__global__ void __launch_bounds__(128)
attn_latent_merge_kernel(const float* __restrict__ partials, const int* __restrict__ tok_slot, __nv_bfloat16* __restrict__ out,
                         int ld_out, int H, int C, int n_split) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    const int tok = blockIdx.x, h = blockIdx.y;
    const int hgs = (H + 15) / 16, hg = h >> 4, r = h & 15;
    __nv_bfloat16* dst = out + (size_t)tok * ld_out + (size_t)h * C;
    if (tok_slot[tok] < 0) {
        for (int c = threadIdx.x; c < C; c += 128) dst[c] = __float2bfloat16_rn(0.f);
        return;
    }
    const float* base = partials + ((size_t)tok * hgs + hg) * n_split * 16 * (C + 2) + (size_t)r * (C + 2);
    const size_t stride = (size_t)16 * (C + 2);
    float m = -INFINITY;
    for (int s = 0; s < n_split; ++s) m = fmaxf(m, base[s * stride + C]);
    float denom = 0.f;
    for (int s = 0; s < n_split; ++s) {
        const float ms = base[s * stride + C];
        if (ms != -INFINITY) denom += expf(ms - m) * base[s * stride + C + 1];
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = threadIdx.x; c < C; c += 128) {
        float v = 0.f;
        for (int s = 0; s < n_split; ++s) {
            const float ms = base[s * stride + C];
            if (ms != -INFINITY) v += expf(ms - m) * base[s * stride + c];
        }
        dst[c] = __float2bfloat16_rn(v * inv);
    }
}

size_t lm_smem_bytes(int G, int D) {
    return ((size_t)G * 16 + 2 * LM_KT) * (D + 8) * 2 + (size_t)G * 2 * 16 * (LM_KT + LM_SPAD) * 4;
}
}  // namespace

// Whether the tensor-core kernel takes these sizes (bfloat16 only).
extern "C" int vlrf_attn_latent_mma_takes(int C, int R, int row_w, int BT, int ld_q) {
    if (C < 32 || C % 32 != 0 || C > 32 * LM_NT_MAX || R < 0 || R % 16 != 0) return 0;
    if (row_w < C + R || row_w % 8 != 0 || BT % LM_KT != 0 || ld_q % 8 != 0) return 0;
    return lm_smem_bytes(1, C + R) <= 200 * 1024 ? 1 : 0;
}
// float32 scratch that n_split > 1 wants
extern "C" long long vlrf_attn_latent_mma_scratch_floats(int n_tokens, int H, int C, int n_split) {
    return (long long)n_tokens * ((H + 15) / 16) * n_split * 16 * (C + 2);
}
// CTAs of a decode step (one token group each) that an SM holds at a time, by their shared memory and warps.
extern "C" int vlrf_attn_latent_mma_ctas_per_sm(int C, int R) {
    const size_t each = lm_smem_bytes(1, C + R) + 1024;
    const int by_smem = (int)((size_t)227 * 1024 / each);
    return by_smem < 1 ? 1 : (by_smem > 16 ? 16 : by_smem);
}
// Tokens a CTA of a prompt step: the most whose queries fit beside the tiles.
extern "C" int vlrf_attn_latent_mma_group(int C, int R) {
    return lm_smem_bytes(4, C + R) <= 200 * 1024 ? 4 : 1;
}

extern "C" int vlrf_attn_latent_mma(const void* qp, int ld_q, const void* cache, int row_w, int C, int R,
                                    const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                                    const int* seq_pos0, void* out, int ld_out, int n_seqs, int max_new, int H, int BT,
                                    float scale, int window, int n_split, float* partials, int* dev_err,
                                    cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_latent_mma_takes(C, R, row_w, BT, ld_q), "attn_latent_mma: does not take C=%d R=%d row=%d BT=%d ld_q=%d", C, R, row_w, BT, ld_q);
    VLRF_REQUIRE(n_seqs >= 0 && max_new >= 1 && H > 0 && max_blocks > 0 && window >= 0 && dev_err != nullptr, "attn_latent_mma: bad arguments");
    VLRF_REQUIRE(ld_q >= H * (C + R) && ld_out >= H * C && ld_out % 2 == 0, "attn_latent_mma: leading sizes are too small");
    VLRF_REQUIRE(n_split >= 1 && n_split <= 64 && (n_split == 1 || (max_new == 1 && partials != nullptr)),
                 "attn_latent_mma: contexts are cut into parts only in decode steps, and parts need scratch");
    if (n_seqs == 0) return VLRF_OK;
    const int hgs = (H + 15) / 16;
    const int G = max_new > 1 ? vlrf_attn_latent_mma_group(C, R) : 1;
    const int tiles_per_seq = (max_new + G - 1) / G;
    dim3 grid((unsigned)(n_seqs * tiles_per_seq), hgs, n_split);
    const size_t smem = lm_smem_bytes(G, C + R);
    auto kern = G == 4 ? attn_latent_mma_kernel<4> : attn_latent_mma_kernel<1>;
    static bool raised[2] = {false, false};
    if (!raised[G == 4]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_latent_mma: shared memory: %s", cudaGetErrorString(e));
        raised[G == 4] = true;
    }
    launch_chained(kern, dim3(grid), dim3(G * 128), (size_t)(smem), stream, (const __nv_bfloat16*)qp, ld_q, (const __nv_bfloat16*)cache, row_w, C, R, block_table,
                                          max_blocks, seq_slot, seq_start, seq_pos0, tiles_per_seq, (__nv_bfloat16*)out, ld_out, H,
                                          BT, scale, window, n_split, partials, dev_err);
    int st = vlrf_check_launch("attn_latent_mma");
    if (st != VLRF_OK || n_split == 1) return st;
    launch_chained(attn_latent_merge_kernel, dim3(dim3(n_seqs, H)), dim3(128), (size_t)(0), stream, partials, seq_slot, (__nv_bfloat16*)out, ld_out, H, C, n_split);
    return vlrf_check_launch("attn_latent_merge");
}
