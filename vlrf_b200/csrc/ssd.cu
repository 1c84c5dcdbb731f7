// A selective state-space recurrence with a matrix state per head, and the kernels around it.
//
// Per sequence and head the state S is N × P float32 (N: state size, P: the head's value size).  A token brings a
// value x (P numbers), an input vector B and an output vector C (N numbers each, shared by the heads of a group) and a
// step size dt > 0:
//     S ← exp(−exp(a_log) · dt) · S + dt · B xᵀ,          y = Sᵀ C + D · x.
// Everything of the recurrence is float32: the state, decay, step size (softplus of the projected number plus a bias,
// unclamped), exponentials.
//
// What a sequence keeps between steps lies in one float32 row per (layer, slot), twice: [2][H·N·P + (taps−1)·channels],
// the state of every head and the last taps − 1 inputs of the short convolution.  A step reads the copy whose index
// is the parity of the sequence's position at the step's start and writes the copy of the parity at its end, so a
// step of one token (or any odd number) leaves what it read untouched and may be run again with the same result.
//
//   ssd_conv        causal convolution per channel over the float32 projection's columns (zeros, or the kept inputs,
//                   before the step's first token), bias, x·sigmoid(x); one thread per channel and run of 64 tokens
//   ssd_conv_state  the last taps − 1 inputs of every sequence into the copy the step writes
//   ssd_scan        the recurrence, token by token: a CTA per (head, sequence), the state in registers (thread (p, j)
//                   holds the rows j, j + NS, … of column p), C-weighted column sums over the NS threads of a column
//                   through shared memory; serves prompts and single tokens alike
//   ssd_gate_norm   y · (z·sigmoid(z)), RMS norm in equal groups, weight, a factor; rounded to the activation dtype
#include "common.cuh"

namespace {
constexpr int CONV_RUN = 64;
constexpr int CONV_MAX_TAPS = 16;

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__global__ void __launch_bounds__(128)
ssd_conv_kernel(const float* __restrict__ proj, int ld, int x_off, const float* __restrict__ w, const float* __restrict__ bias,
                const float* __restrict__ state, int state_row, int conv_off, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, float* __restrict__ out, int channels,
                int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    const int slot = seq_slot[s];
    if (c >= channels || slot < 0) return;
    const int start = seq_start[s], n = seq_start[s + 1] - start;
    const int i0 = blockIdx.z * CONV_RUN;
    if (i0 >= n) return;
    const int i1 = min(n, i0 + CONV_RUN);
    const float* kept = state + ((size_t)slot * 2 + (seq_pos0[s] & 1)) * state_row + conv_off;   // [taps − 1][channels]
    float wt[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    const float b = bias[c];
    for (int i = i0; i < i1; ++i) {
        float acc = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j < taps) {
                const int ii = i - (taps - 1) + j;
                const float v = ii >= 0 ? proj[(size_t)(start + ii) * ld + x_off + c] : kept[(size_t)(taps - 1 + ii) * channels + c];
                acc = fmaf(wt[j], v, acc);
            }
        }
        out[(size_t)(start + i) * channels + c] = silu_f(acc);
    }
}

__global__ void __launch_bounds__(128)
ssd_conv_state_kernel(const float* __restrict__ proj, int ld, int x_off, float* __restrict__ state, int state_row, int conv_off,
                      const int* __restrict__ seq_slot, const int* __restrict__ seq_start, const int* __restrict__ seq_pos0,
                      int channels, int taps) {
    pdl_wait();
    pdl_launch_dependents();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    const int slot = seq_slot[s];
    if (c >= channels || slot < 0) return;
    const int start = seq_start[s], n = seq_start[s + 1] - start, pos0 = seq_pos0[s];
    const float* kept = state + ((size_t)slot * 2 + (pos0 & 1)) * state_row + conv_off;
    float* next = state + ((size_t)slot * 2 + ((pos0 + n) & 1)) * state_row + conv_off;
    float v[CONV_MAX_TAPS];
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k) {
        if (k < taps - 1) {
            const int ii = n - (taps - 1) + k;
            v[k] = ii >= 0 ? proj[(size_t)(start + ii) * ld + x_off + c] : kept[(size_t)(taps - 1 + ii) * channels + c];
        }
    }
#pragma unroll
    for (int k = 0; k < CONV_MAX_TAPS; ++k)
        if (k < taps - 1) next[(size_t)k * channels + c] = v[k];
}

// R: rows of the state a thread holds.  blockDim = P · NS; thread (p = tid % P, j = tid / P).
template <int R>
__global__ void __launch_bounds__(256)
ssd_scan_kernel(const float* __restrict__ xbc, int channels, const float* __restrict__ proj, int ld, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ Dv,
                float* __restrict__ state, int state_row, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                const int* __restrict__ seq_pos0, float* __restrict__ y, int Hs, int G, int N, int P, int NS) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float red[];          // [2][NS][P]
    const int h = blockIdx.x, s = blockIdx.y;
    const int slot = seq_slot[s];
    if (slot < 0) return;
    const int start = seq_start[s], n = seq_start[s + 1] - start, pos0 = seq_pos0[s];
    const int p = threadIdx.x % P, j = threadIdx.x / P;
    const int inner = Hs * P, g = h / (Hs / G);
    const float* S_in = state + ((size_t)slot * 2 + (pos0 & 1)) * state_row + (size_t)h * N * P;
    float* S_out = state + ((size_t)slot * 2 + ((pos0 + n) & 1)) * state_row + (size_t)h * N * P;
    float S[R];
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = j + k * NS;
        S[k] = r < N ? S_in[(size_t)r * P + p] : 0.f;
    }
    const float a = -expf(a_log[h]), dtb = dt_bias[h], dh = Dv[h];
    const int b_off = inner + g * N, c_off = inner + G * N + g * N;
    for (int i = 0; i < n; ++i) {
        const size_t row = (size_t)(start + i);
        const float* xr = xbc + row * channels;
        const float dt = softplus_f(proj[row * ld + dt_off + h] + dtb);
        const float decay = expf(a * dt);
        const float xv = xr[h * P + p];
        const float dx = dt * xv;
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < R; ++k) {
            const int r = j + k * NS;
            if (r < N) {
                S[k] = fmaf(decay, S[k], xr[b_off + r] * dx);
                part = fmaf(S[k], xr[c_off + r], part);
            }
        }
        float* buf = red + (size_t)(i & 1) * NS * P;
        buf[j * P + p] = part;
        __syncthreads();
        if (j == 0) {
            float sum = 0.f;
            for (int q = 0; q < NS; ++q) sum += buf[q * P + p];
            y[row * inner + h * P + p] = fmaf(dh, xv, sum);
        }
    }
#pragma unroll
    for (int k = 0; k < R; ++k) {
        const int r = j + k * NS;
        if (r < N) S_out[(size_t)r * P + p] = S[k];
    }
}

template <typename OT>
__global__ void __launch_bounds__(128)
ssd_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ proj, int ld, int z_off, const float* __restrict__ w,
                     OT* __restrict__ out, int ld_out, int d, int groups, float eps, float factor) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float v_sm[];          // [d], then [groups]
    float* inv_sm = v_sm + d;
    const int r = blockIdx.x;
    const float* yr = y + (size_t)r * d;
    const float* zr = proj + (size_t)r * ld + z_off;
    for (int i = threadIdx.x; i < d; i += blockDim.x) v_sm[i] = yr[i] * silu_f(zr[i]);
    __syncthreads();
    const int gs = d / groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < groups; g += blockDim.x / 32) {
        float ss = 0.f;
        for (int i = lane; i < gs; i += 32) { const float v = v_sm[g * gs + i]; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        if (lane == 0) inv_sm[g] = factor / sqrtf(ss / (float)gs + eps);
    }
    __syncthreads();
    OT* o = out + (size_t)r * ld_out;
    for (int i = threadIdx.x; i < d; i += blockDim.x) ElemIO<OT>::store(o + i, v_sm[i] * inv_sm[i / gs] * w[i]);
}
}  // namespace

extern "C" int vlrf_ssd_conv(const float* proj, int ld, int x_off, const float* w, const float* bias, float* state, int state_row,
                             int conv_off, const int* seq_slot, const int* seq_start, const int* seq_pos0, float* out, int n_seqs,
                             int max_new, int channels, int taps, cudaStream_t stream) {
    VLRF_REQUIRE(n_seqs >= 0 && max_new >= 0 && channels > 0, "ssd_conv: bad sizes");
    VLRF_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "ssd_conv: %d taps are not in 1…%d", taps, CONV_MAX_TAPS);
    VLRF_REQUIRE(x_off + channels <= ld && conv_off + (taps - 1) * channels <= state_row, "ssd_conv: columns lie outside the row");
    if (n_seqs == 0 || max_new == 0) return VLRF_OK;
    const dim3 grid((channels + 127) / 128, n_seqs, (max_new + CONV_RUN - 1) / CONV_RUN);
    launch_chained(ssd_conv_kernel, grid, dim3(128), (size_t)0, stream, proj, ld, x_off, w, bias, (const float*)state, state_row,
                   conv_off, seq_slot, seq_start, seq_pos0, out, channels, taps);
    if (vlrf_check_launch("ssd_conv") != VLRF_OK) return VLRF_ERR_CUDA;
    if (taps > 1) {
        launch_chained(ssd_conv_state_kernel, dim3((channels + 127) / 128, n_seqs), dim3(128), (size_t)0, stream, proj, ld, x_off,
                       state, state_row, conv_off, seq_slot, seq_start, seq_pos0, channels, taps);
        return vlrf_check_launch("ssd_conv_state");
    }
    return VLRF_OK;
}

extern "C" int vlrf_ssd_scan(const float* xbc, int channels, const float* proj, int ld, int dt_off, const float* dt_bias,
                             const float* a_log, const float* D, float* state, int state_row, const int* seq_slot,
                             const int* seq_start, const int* seq_pos0, float* y, int n_seqs, int Hs, int G, int N, int P,
                             cudaStream_t stream) {
    VLRF_REQUIRE(n_seqs >= 0 && Hs > 0 && G > 0 && N > 0 && P > 0, "ssd_scan: bad sizes");
    VLRF_REQUIRE(Hs % G == 0, "ssd_scan: %d heads cannot share %d groups", Hs, G);
    VLRF_REQUIRE(P <= 256, "ssd_scan: a head's value size of %d is above 256", P);
    VLRF_REQUIRE(channels == Hs * P + 2 * G * N && dt_off + Hs <= ld && (size_t)Hs * N * P <= (size_t)state_row,
                 "ssd_scan: the rows do not hold what the sizes say");
    if (n_seqs == 0) return VLRF_OK;
    const int NS = 256 / P > 0 ? (256 / P < N ? 256 / P : N) : 1;
    const int rows = (N + NS - 1) / NS;
    VLRF_REQUIRE(rows <= 128, "ssd_scan: a state of %d rows by %d columns is larger than a CTA's registers hold", N, P);
    const dim3 grid(Hs, n_seqs), block(P * NS);
    const size_t smem = (size_t)2 * NS * P * sizeof(float);
#define GO(R) launch_chained(ssd_scan_kernel<R>, grid, block, smem, stream, xbc, channels, proj, ld, dt_off, dt_bias, a_log, D, state, \
                             state_row, seq_slot, seq_start, seq_pos0, y, Hs, G, N, P, NS)
    if (rows <= 8) GO(8);
    else if (rows <= 16) GO(16);
    else if (rows <= 32) GO(32);
    else if (rows <= 64) GO(64);
    else GO(128);
#undef GO
    return vlrf_check_launch("ssd_scan");
}

extern "C" int vlrf_ssd_gate_norm(const float* y, const float* proj, int ld, int z_off, const float* w, void* out, int out_dtype,
                                  int ld_out, int n_rows, int d, int groups, float eps, float factor, cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && d > 0 && groups > 0 && d % groups == 0, "ssd_gate_norm: %d columns in %d groups", d, groups);
    VLRF_REQUIRE(z_off + d <= ld && ld_out >= d, "ssd_gate_norm: columns lie outside the row");
    const size_t smem = (size_t)(d + groups) * sizeof(float);
    VLRF_REQUIRE(smem <= 160 * 1024, "ssd_gate_norm: a row of %d numbers does not fit shared memory", d);
    if (n_rows == 0) return VLRF_OK;
    if (out_dtype == VLRF_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ssd_gate_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(ssd_gate_norm_kernel<float>, dim3(n_rows), dim3(128), smem, stream, y, proj, ld, z_off, w, (float*)out, ld_out, d,
                       groups, eps, factor);
    } else if (out_dtype == VLRF_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(ssd_gate_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(ssd_gate_norm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(128), smem, stream, y, proj, ld, z_off, w,
                       (__nv_bfloat16*)out, ld_out, d, groups, eps, factor);
    } else {
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "ssd_gate_norm: unknown output dtype %d", out_dtype);
    }
    return vlrf_check_launch("ssd_gate_norm");
}
