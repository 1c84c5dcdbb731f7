// Prompt attention over keys and values that lie in plain rows (bfloat16, `mma.sync`), for steps in which every
// sequence begins at its first token, so that all keys and values of the step are the step's own.
//
// A mixer whose cache holds something else than keys and values (a latent from which they are linear maps) forms them
// for such a step with two ordinary products and calls this kernel; steps that go on from a cache take the mixer's
// other path.  Queries and keys have two parts that are stored apart: a part per head (dim columns: qn [T][H·dim],
// kn [T][H·dim]) and a part whose key all heads share (R columns: qr [T][H·R], kr [T][≥ R] with a row stride of its
// own; R may be 0).  The score of query i and key j ≤ i of the same sequence is (qn_h(i)·kn_h(j) + qr_h(i)·kr(j))·scale;
// softmax in float32; values v [T][H·vdim]; out [T][H·vdim].
//
// A CTA takes 64 consecutive queries of one sequence and one head: four warps of 16 query rows each, whose MMA
// operands stay in registers.  Tiles of 32 keys ([kn | kr] rows) and values arrive by `cp.async` in two buffers;
// a warp multiplies its queries by the tile, keeps maximum and sum of its rows in registers, and adds P·V to its
// accumulators (the scores' fragments are the next MMA's operands as they are).  Tiles wholly above a warp's rows are
// skipped.  Sizes: dim + R one of 32, 64, 96, 128, 192, 256; dim and R multiples of 8; vdim a multiple of 8 up to 128.
#include "common.cuh"

namespace {
constexpr int AR_QT = 64, AR_KT = 32, AR_NT_MAX = 16;

__device__ __forceinline__ uint32_t ar_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ar_ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ar_ldsm_x2_trans(uint32_t& r0, uint32_t& r1, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void ar_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ar_cp16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t ar_pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// KQ: 16-column steps of dim + R
template <int KQ>
__global__ void __launch_bounds__(128)
attn_rows_kernel(const __nv_bfloat16* __restrict__ qn, int ld_qn, const __nv_bfloat16* __restrict__ qr, int ld_qr,
                 const __nv_bfloat16* __restrict__ kn, int ld_kn, const __nv_bfloat16* __restrict__ kr, int ld_kr,
                 const __nv_bfloat16* __restrict__ v, int ld_v, const int* __restrict__ seq_start, int n_seqs, int tiles_per_seq,
                 __nv_bfloat16* __restrict__ out, int ld_out, int dim, int R, int vdim, float scale) {
    pdl_wait();                 // chained launch: nothing is read before the kernels ahead have finished
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char ar_raw[];
    constexpr int DK = KQ * 16, LDK = DK + 8;
    const int ldv = vdim + 8;
    __nv_bfloat16* k_sm = reinterpret_cast<__nv_bfloat16*>(ar_raw);                    // [2][AR_KT][LDK]; first the queries [64][LDK]
    __nv_bfloat16* v_sm = k_sm + (size_t)2 * AR_KT * LDK;                              // [2][AR_KT][ldv]
    const int tid = threadIdx.x, w = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    // (the tiles of late queries have the most keys: they come first in the grid, so that the short ones fill the end)
    const int seq = blockIdx.x % n_seqs, q0 = (tiles_per_seq - 1 - blockIdx.x / n_seqs) * AR_QT, h = blockIdx.y;
    const int row0 = seq_start[seq], len = seq_start[seq + 1] - row0;
    if (q0 >= len) return;
    const int q_last = min(q0 + AR_QT, len) - 1;                   // last query of the CTA = last key it needs
    // the CTA's queries [qn | qr] into shared memory (the place of the first tile pair), then each warp's 16 rows into
    // registers as MMA operands
    for (int i = tid; i < AR_QT * (DK / 8); i += 128) {
        const int r = i / (DK / 8), c = (i - r * (DK / 8)) * 8;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        if (q0 + r < len) {
            const size_t row = (size_t)(row0 + q0 + r);
            x = c < dim ? *reinterpret_cast<const uint4*>(qn + row * ld_qn + (size_t)h * dim + c)
                        : *reinterpret_cast<const uint4*>(qr + row * ld_qr + (size_t)h * R + (c - dim));
        }
        *reinterpret_cast<uint4*>(k_sm + (size_t)r * LDK + c) = x;
    }
    __syncthreads();
    uint32_t aq[KQ][4];
    {
        const uint32_t a_addr = ar_smem(k_sm) + (uint32_t)((16 * w + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDK + 8 * (lane >> 4)) * 2;
#pragma unroll
        for (int j = 0; j < KQ; ++j) ar_ldsm_x4(aq[j], a_addr + j * 32);
    }
    __syncthreads();                                               // the queries' place becomes the tiles'
    const int chunks_k = DK / 8, chunks_v = vdim / 8;
    auto fetch = [&](int tile, int buf) {
        const int key0 = tile * AR_KT;
        __nv_bfloat16* kd = k_sm + (size_t)buf * AR_KT * LDK;
        __nv_bfloat16* vd = v_sm + (size_t)buf * AR_KT * ldv;
        for (int i = tid; i < AR_KT * chunks_k; i += 128) {
            const int r = i / chunks_k, c = (i - r * chunks_k) * 8;
            const bool live = key0 + r <= q_last;                  // rows nobody may see arrive as zeros
            const size_t row = (size_t)(row0 + (live ? key0 + r : 0));
            const __nv_bfloat16* src = c < dim ? kn + row * ld_kn + (size_t)h * dim + c : kr + row * ld_kr + (c - dim);
            ar_cp16(ar_smem(kd + (size_t)r * LDK + c), src, live ? 16 : 0);
        }
        for (int i = tid; i < AR_KT * chunks_v; i += 128) {
            const int r = i / chunks_v, c = (i - r * chunks_v) * 8;
            const bool live = key0 + r <= q_last;
            const size_t row = (size_t)(row0 + (live ? key0 + r : 0));
            ar_cp16(ar_smem(vd + (size_t)r * ldv + c), v + row * ld_v + (size_t)h * vdim + c, live ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int n_tiles = q_last / AR_KT + 1;
    const int my_q0 = q0 + 16 * w;                                 // this warp's rows: my_q0 + g and my_q0 + g + 8
    const int nt_cnt = vdim >> 3;
    float acc[AR_NT_MAX][4];
#pragma unroll
    for (int i = 0; i < AR_NT_MAX; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    fetch(0, 0);
    for (int tile = 0; tile < n_tiles; ++tile) {
        const int buf = tile & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                           // the tile has landed; the other buffer is free
        if (tile + 1 < n_tiles) fetch(tile + 1, buf ^ 1);
        const int key0 = tile * AR_KT;
        if (key0 > my_q0 + 15 || my_q0 >= len) continue;           // wholly above this warp's rows, or no rows at all
        const __nv_bfloat16* kt = k_sm + (size_t)buf * AR_KT * LDK;
        const __nv_bfloat16* vt = v_sm + (size_t)buf * AR_KT * ldv;
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
        // one ldmatrix: (keys 0-7, k lo), (keys 0-7, k hi), (keys 8-15, k lo), (keys 8-15, k hi) of a k-step
        const uint32_t b_addr = ar_smem(kt) + (uint32_t)(((lane & 7) + 8 * (lane >> 4)) * LDK + 8 * ((lane >> 3) & 1)) * 2;
#pragma unroll
        for (int j = 0; j < KQ; ++j) {
            uint32_t b0[4], b1[4];
            ar_ldsm_x4(b0, b_addr + j * 32);
            ar_ldsm_x4(b1, b_addr + (uint32_t)(16 * LDK) * 2 + j * 32);
            ar_mma(s[0], aq[j], b0[0], b0[1]);
            ar_mma(s[1], aq[j], b0[2], b0[3]);
            ar_mma(s[2], aq[j], b1[0], b1[1]);
            ar_mma(s[3], aq[j], b1[2], b1[3]);
        }
        // scale and mask: s[nt][e]: row g (e < 2) or g + 8, key key0 + 8·nt + 2·t4 + (e & 1)
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 4; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + 8 * nt + 2 * t4 + (e & 1), q = my_q0 + g + 8 * (e >> 1);
                s[nt][e] = key <= q ? s[nt][e] * scale : -INFINITY;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;   // a row that sees nothing of the tile (it lies behind the sequence)
            corr[r] = m_run[r] == -INFINITY ? 0.f : expf(m_run[r] - m_use);
            float sum = 0.f;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 2 * r; e < 2 * r + 2; ++e) {
                    const float p = __bfloat162float(__float2bfloat16_rn(expf(s[nt][e] - m_use)));   // what the MMA multiplies
                    s[nt][e] = p;
                    sum += p;
                }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            l_run[r] = l_run[r] * corr[r] + sum;
            m_run[r] = m_new;
        }
        uint32_t pa[2][4];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            pa[kk][0] = ar_pack(s[2 * kk][0], s[2 * kk][1]);
            pa[kk][1] = ar_pack(s[2 * kk][2], s[2 * kk][3]);
            pa[kk][2] = ar_pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
            pa[kk][3] = ar_pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
        }
#pragma unroll
        for (int nt = 0; nt < AR_NT_MAX; ++nt) {
            if (nt < nt_cnt) { acc[nt][0] *= corr[0]; acc[nt][1] *= corr[0]; acc[nt][2] *= corr[1]; acc[nt][3] *= corr[1]; }
        }
        const uint32_t v_addr = ar_smem(vt) + (uint32_t)(((lane & 7) + 8 * ((lane >> 3) & 1)) * ldv) * 2;
#pragma unroll
        for (int nt0 = 0; nt0 < AR_NT_MAX; nt0 += 4) {
            if (nt0 < nt_cnt) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    uint32_t b[4][2];
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (nt0 + i < nt_cnt) ar_ldsm_x2_trans(b[i][0], b[i][1], v_addr + (uint32_t)(16 * kk * ldv + (nt0 + i) * 8) * 2);
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (nt0 + i < nt_cnt) ar_mma(acc[nt0 + i], pa[kk], b[i][0], b[i][1]);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int q = my_q0 + g + 8 * r;
        if (q >= len) continue;
        const float inv = l_run[r] > 0.f ? 1.f / l_run[r] : 0.f;
        __nv_bfloat16* dst = out + (size_t)(row0 + q) * ld_out + (size_t)h * vdim;
#pragma unroll
        for (int nt = 0; nt < AR_NT_MAX; ++nt)
            if (nt < nt_cnt) *reinterpret_cast<uint32_t*>(dst + nt * 8 + 2 * t4) = ar_pack(acc[nt][2 * r] * inv, acc[nt][2 * r + 1] * inv);
    }
}

size_t ar_smem_bytes(int dk, int vdim) {
    const size_t tiles = (size_t)2 * AR_KT * (dk + 8) * 2 + (size_t)2 * AR_KT * (vdim + 8) * 2;
    const size_t queries = (size_t)AR_QT * (dk + 8) * 2;
    return tiles > queries ? tiles : queries;
}
}  // namespace

extern "C" int vlrf_attn_rows_takes(int dim, int R, int vdim, int ld_qn, int ld_qr, int ld_kn, int ld_kr, int ld_v, int ld_out) {
    const int dk = dim + R;
    if (!(dk == 32 || dk == 64 || dk == 96 || dk == 128 || dk == 192 || dk == 256)) return 0;
    if (dim < 8 || dim % 8 != 0 || R < 0 || R % 8 != 0 || vdim < 8 || vdim % 8 != 0 || vdim > 8 * AR_NT_MAX) return 0;
    if (ld_qn % 8 != 0 || (R > 0 && (ld_qr % 8 != 0 || ld_kr % 8 != 0)) || ld_kn % 8 != 0 || ld_v % 8 != 0 || ld_out % 2 != 0) return 0;
    return 1;
}

extern "C" int vlrf_attn_rows(const void* qn, int ld_qn, const void* qr, int ld_qr, const void* kn, int ld_kn, const void* kr,
                              int ld_kr, const void* v, int ld_v, const int* seq_start, void* out, int ld_out, int n_seqs,
                              int max_new, int H, int dim, int R, int vdim, float scale, cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_rows_takes(dim, R, vdim, ld_qn, ld_qr, ld_kn, ld_kr, ld_v, ld_out), "attn_rows: does not take dim=%d R=%d vdim=%d", dim, R, vdim);
    VLRF_REQUIRE(n_seqs >= 0 && max_new >= 1 && H > 0 && H <= 65535 && seq_start != nullptr, "attn_rows: bad arguments");
    VLRF_REQUIRE(((reinterpret_cast<uintptr_t>(qn) | reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(v) |
                   reinterpret_cast<uintptr_t>(qr) | reinterpret_cast<uintptr_t>(kr)) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 3) == 0,
                 "attn_rows: rows must start on 16-byte boundaries");
    if (n_seqs == 0) return VLRF_OK;
    const int tiles_per_seq = (max_new + AR_QT - 1) / AR_QT;
    const dim3 grid((unsigned)(n_seqs * tiles_per_seq), H);
    const size_t smem = ar_smem_bytes(dim + R, vdim);
#define AR_GO(KQ)                                                                                                              \
    {                                                                                                                          \
        static bool raised = false;                                                                                            \
        if (!raised) {                                                                                                         \
            cudaError_t e = cudaFuncSetAttribute(attn_rows_kernel<KQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024); \
            if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_rows: shared memory: %s", cudaGetErrorString(e));      \
            raised = true;                                                                                                     \
        }                                                                                                                      \
        launch_chained(attn_rows_kernel<KQ>, grid, dim3(128), smem, stream, (const __nv_bfloat16*)qn, ld_qn, (const __nv_bfloat16*)qr, \
                       ld_qr, (const __nv_bfloat16*)kn, ld_kn, (const __nv_bfloat16*)kr, ld_kr, (const __nv_bfloat16*)v, ld_v,  \
                       seq_start, n_seqs, tiles_per_seq, (__nv_bfloat16*)out, ld_out, dim, R, vdim, scale);                            \
    }
    switch ((dim + R) / 16) {
        case 2: AR_GO(2) break;
        case 4: AR_GO(4) break;
        case 6: AR_GO(6) break;
        case 8: AR_GO(8) break;
        case 12: AR_GO(12) break;
        default: AR_GO(16) break;
    }
#undef AR_GO
    return vlrf_check_launch("attn_rows");
}
