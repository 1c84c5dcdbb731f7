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
//                   before the step's first token), bias, x·sigmoid(x); one thread per channel and run of 16 tokens
//   ssd_conv_state  the last taps − 1 inputs of every sequence into the copy the step writes
//   ssd_scan        the recurrence, token by token: a CTA per (head, 32 columns of the state, sequence), a lane per
//                   column, a warp per slice of rows, the state in registers; the inputs of 16 tokens at a time arrive in
//                   shared memory by `cp.async` a batch ahead, B and C are read from there by every lane alike; the
//                   C-weighted sums of the slices meet in shared memory once per batch;
//                   serves prompts and single tokens alike, with the same arithmetic in the same order
//   ssd_gate_norm   y · (z·sigmoid(z)), RMS norm in equal groups, weight, a factor; rounded to the activation dtype
#include "common.cuh"

namespace {
constexpr int CONV_RUN = 16;
constexpr int CONV_MAX_TAPS = 16;

__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

__global__ void __launch_bounds__(128)
ssd_conv_kernel(const float* __restrict__ proj, int ld, int x_off, const float* __restrict__ w, const float* __restrict__ bias,
                const float* __restrict__ state, int state_row, int conv_off, const int* __restrict__ seq_slot,
                const int* __restrict__ seq_start, const int* __restrict__ seq_pos0, float* __restrict__ out, int channels,
                int taps, float* __restrict__ keep) {
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
    // the taps and the last taps − 1 inputs in registers: every input of the run is read once
    float wt[CONV_MAX_TAPS], win[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        win[j] = 0.f;
        if (j < taps - 1) {
            const int ii = i0 - (taps - 1) + j;
            win[j] = ii >= 0 ? proj[(size_t)(start + ii) * ld + x_off + c] : kept[(size_t)(taps - 1 + ii) * channels + c];
        }
    }
    const float b = bias[c], w_cur = w[(size_t)c * taps + taps - 1];
    // the run's inputs are asked for together, ahead of the sums that use them one after another
    float in[CONV_RUN];
#pragma unroll
    for (int k = 0; k < CONV_RUN; ++k) in[k] = (i0 + k < i1) ? proj[(size_t)(start + i0 + k) * ld + x_off + c] : 0.f;
#pragma unroll
    for (int k = 0; k < CONV_RUN; ++k) {
        const int i = i0 + k;
        if (i >= i1) break;
        const float cur = in[k];
        float acc = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
            if (j < taps - 1) {
                acc = fmaf(wt[j], win[j], acc);
                win[j] = (j + 1 < taps - 1) ? win[j + 1] : cur;
            }
        }
        acc = fmaf(w_cur, cur, acc);
        out[(size_t)(start + i) * channels + c] = silu_f(acc);
    }
    // keep != null (every sequence is one run: this thread alone has read the channel's kept inputs): the last taps − 1
    // inputs into the copy that the step writes, which may be the copy it read
    if (keep != nullptr) {
        float* next = keep + ((size_t)slot * 2 + ((seq_pos0[s] + n) & 1)) * state_row + conv_off;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j)
            if (j < taps - 1) next[(size_t)j * channels + c] = win[j];
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

// NR: rows of the state a warp holds (one column a lane).  A CTA is (head, block of 32 columns, sequence); its warps
// are the slices of NR rows.  The columns of a state never meet, so nothing but the C-weighted sums over the slices
// crosses warps: those go through shared memory once per batch of up to 16 tokens.
constexpr int SC_MAX_BATCH = 16;

__device__ __forceinline__ void sc_cp4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void sc_cp16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int NR, bool VEC>
__global__ void __launch_bounds__(512)
ssd_scan_kernel(const float* __restrict__ xbc, int channels, const float* __restrict__ proj, int ld, int dt_off,
                const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ Dv,
                float* __restrict__ state, int state_row, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                const int* __restrict__ seq_pos0, float* __restrict__ y, int Hs, int G, int N, int P, int PB, int SC_BATCH) {
    pdl_wait();
    pdl_launch_dependents();
    // shared memory: the C-weighted sums of the slices [2][SC_BATCH][slices][32], then per stage the batch's inputs:
    // x [SC_BATCH][32], B [SC_BATCH][NP], C [SC_BATCH][NP] (NP: N rounded up to a multiple of 4; SC_BATCH: tokens a
    // batch, at most 16, fewer where no sequence brings as many)
    extern __shared__ __align__(16) float sc_sm[];
    const int h = blockIdx.x / PB, pb = blockIdx.x - h * PB, s = blockIdx.y;
    const int slot = seq_slot[s];
    if (slot < 0) return;
    const int start = seq_start[s], n = seq_start[s + 1] - start, pos0 = seq_pos0[s];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, slices = blockDim.x >> 5;
    const int NP = (N + 3) & ~3, stage_floats = SC_BATCH * (32 + 2 * NP);
    float* part_sm = sc_sm;
    float* in_sm = sc_sm + 2 * SC_BATCH * slices * 32;
    const int p = pb * 32 + lane, n0 = warp * NR;
    const bool col = p < P;
    const int inner = Hs * P, g = h / (Hs / G);
    const float* S_in = state + ((size_t)slot * 2 + (pos0 & 1)) * state_row + (size_t)h * N * P;
    float* S_out = state + ((size_t)slot * 2 + ((pos0 + n) & 1)) * state_row + (size_t)h * N * P;
    float S[NR];
#pragma unroll
    for (int k = 0; k < NR; ++k) S[k] = (col && n0 + k < N) ? S_in[(size_t)(n0 + k) * P + p] : 0.f;
    const float a = -expf(a_log[h]), dtb = dt_bias[h], dh = Dv[h];
    const int b_col = inner + g * N, c_col = inner + G * N + g * N, x_col = h * P + pb * 32;
    const int n_x = min(32, P - pb * 32);

    auto fetch = [&](int i0, int stage) {       // all threads: the inputs of the batch that begins at token i0
        const int nb = min(SC_BATCH, n - i0);
        float* xs = in_sm + stage * stage_floats;
        float* bs = xs + SC_BATCH * 32;
        float* cs = bs + SC_BATCH * NP;
        for (int idx = threadIdx.x; idx < nb * 32; idx += blockDim.x) {
            const int ii = idx >> 5, l = idx & 31;
            if (l < n_x) sc_cp4(xs + idx, xbc + (size_t)(start + i0 + ii) * channels + x_col + l);
            else xs[idx] = 0.f;
        }
        if (VEC) {
            const int q = N / 4;
            for (int idx = threadIdx.x; idx < nb * q; idx += blockDim.x) {
                const int ii = idx / q, c4 = (idx - ii * q) * 4;
                const float* row = xbc + (size_t)(start + i0 + ii) * channels;
                sc_cp16(bs + ii * NP + c4, row + b_col + c4);
                sc_cp16(cs + ii * NP + c4, row + c_col + c4);
            }
        } else {
            for (int idx = threadIdx.x; idx < nb * N; idx += blockDim.x) {
                const int ii = idx / N, c = idx - ii * N;
                const float* row = xbc + (size_t)(start + i0 + ii) * channels;
                sc_cp4(bs + ii * NP + c, row + b_col + c);
                sc_cp4(cs + ii * NP + c, row + c_col + c);
            }
        }
    };
    fetch(0, 0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    float dt_raw = lane < min(SC_BATCH, n) ? proj[(size_t)(start + lane) * ld + dt_off + h] : 0.f;
    for (int i0 = 0, b = 0; i0 < n; i0 += SC_BATCH, ++b) {
        const int nb = min(SC_BATCH, n - i0), buf = b & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                        // the batch's inputs lie in shared memory, and nobody reads the other stage any more
        if (i0 + SC_BATCH < n) fetch(i0 + SC_BATCH, buf ^ 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
        // lane ii works out the step size and the decay of the batch's token ii, and asks for the next batch's number
        const float dt_mine = softplus_f(dt_raw + dtb), decay_mine = expf(a * dt_mine);
        const int nxt = i0 + SC_BATCH + lane;
        dt_raw = nxt < n ? proj[(size_t)(start + nxt) * ld + dt_off + h] : 0.f;
        const float* xs = in_sm + buf * stage_floats;
        const float* xp = xs + lane;
        const float* bs = xs + SC_BATCH * 32 + n0;
        const float* cs = bs + SC_BATCH * NP;
        float* mine = part_sm + ((size_t)buf * SC_BATCH * slices + warp) * 32 + lane;
        const int mine_step = slices * 32;
        const bool whole = n0 + NR <= N;        // (a slice that ends behind the state's last row checks every row)
        if (VEC && whole && nb == SC_MAX_BATCH) {
            // the common case of a prompt, written out for all 16 tokens of a batch: nothing but the loads from shared
            // memory, the two exchanges of step size and decay, and the multiply-adds
#pragma unroll
            for (int ii = 0; ii < SC_MAX_BATCH; ++ii) {
                const float dt = __shfl_sync(0xffffffffu, dt_mine, ii), decay = __shfl_sync(0xffffffffu, decay_mine, ii);
                const float dx = dt * xp[ii * 32];
                const float* bq = bs + ii * NP;
                const float* cq = cs + ii * NP;
                float part0 = 0.f, part1 = 0.f;
#pragma unroll
                for (int k = 0; k < NR; k += 4) {
                    const float4 bv = *reinterpret_cast<const float4*>(bq + k), cv = *reinterpret_cast<const float4*>(cq + k);
                    S[k] = fmaf(decay, S[k], bv.x * dx);         part0 = fmaf(S[k], cv.x, part0);
                    S[k + 1] = fmaf(decay, S[k + 1], bv.y * dx); part1 = fmaf(S[k + 1], cv.y, part1);
                    S[k + 2] = fmaf(decay, S[k + 2], bv.z * dx); part0 = fmaf(S[k + 2], cv.z, part0);
                    S[k + 3] = fmaf(decay, S[k + 3], bv.w * dx); part1 = fmaf(S[k + 3], cv.w, part1);
                }
                mine[ii * mine_step] = part0 + part1;
            }
        } else {
#pragma unroll 2
            for (int ii = 0; ii < nb; ++ii, xp += 32, bs += NP, cs += NP, mine += mine_step) {
                const float dt = __shfl_sync(0xffffffffu, dt_mine, ii), decay = __shfl_sync(0xffffffffu, decay_mine, ii);
                const float dx = dt * xp[0];
                float part0 = 0.f, part1 = 0.f;
                if (VEC && whole) {
#pragma unroll
                    for (int k = 0; k < NR; k += 4) {
                        const float4 bv = *reinterpret_cast<const float4*>(bs + k), cv = *reinterpret_cast<const float4*>(cs + k);
                        S[k] = fmaf(decay, S[k], bv.x * dx);         part0 = fmaf(S[k], cv.x, part0);
                        S[k + 1] = fmaf(decay, S[k + 1], bv.y * dx); part1 = fmaf(S[k + 1], cv.y, part1);
                        S[k + 2] = fmaf(decay, S[k + 2], bv.z * dx); part0 = fmaf(S[k + 2], cv.z, part0);
                        S[k + 3] = fmaf(decay, S[k + 3], bv.w * dx); part1 = fmaf(S[k + 3], cv.w, part1);
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < NR; ++k) {
                        if (n0 + k < N) {
                            S[k] = fmaf(decay, S[k], bs[k] * dx);
                            part0 = fmaf(S[k], cs[k], part0);
                        }
                    }
                }
                mine[0] = part0 + part1;
            }
        }
        __syncthreads();                        // the slices' sums of this batch are complete
        for (int idx = threadIdx.x; idx < nb * 32; idx += blockDim.x) {
            const int ii = idx >> 5, l = idx & 31;
            if (l < n_x) {
                const float* q = part_sm + ((size_t)buf * SC_BATCH + ii) * slices * 32 + l;
                float sum = 0.f;
                for (int w = 0; w < slices; ++w) sum += q[w * 32];
                y[(size_t)(start + i0 + ii) * inner + x_col + l] = fmaf(dh, xs[idx], sum);
            }
        }
        // (the next pass writes the other buffers only behind its first barrier, which this pass's readers reach first)
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
    for (int k = 0; k < NR; ++k)
        if (col && n0 + k < N) S_out[(size_t)(n0 + k) * P + p] = S[k];
}

// (asked of the driver once per instantiation and size: more than 48 KB of shared memory is opt-in)
template <int R, bool V> void scan_allow_smem(size_t smem) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaFuncSetAttribute(ssd_scan_kernel<R, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        allowed = smem;
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
    const bool one_run = max_new <= CONV_RUN;       // then the convolution's threads leave the kept inputs themselves
    launch_chained(ssd_conv_kernel, grid, dim3(128), (size_t)0, stream, proj, ld, x_off, w, bias, (const float*)state, state_row,
                   conv_off, seq_slot, seq_start, seq_pos0, out, channels, taps, (one_run && taps > 1) ? state : (float*)nullptr);
    if (vlrf_check_launch("ssd_conv") != VLRF_OK) return VLRF_ERR_CUDA;
    if (taps > 1 && !one_run) {
        launch_chained(ssd_conv_state_kernel, dim3((channels + 127) / 128, n_seqs), dim3(128), (size_t)0, stream, proj, ld, x_off,
                       state, state_row, conv_off, seq_slot, seq_start, seq_pos0, channels, taps);
        return vlrf_check_launch("ssd_conv_state");
    }
    return VLRF_OK;
}

extern "C" int vlrf_ssd_scan(const float* xbc, int channels, const float* proj, int ld, int dt_off, const float* dt_bias,
                             const float* a_log, const float* D, float* state, int state_row, const int* seq_slot,
                             const int* seq_start, const int* seq_pos0, float* y, int n_seqs, int max_new, int Hs, int G, int N, int P,
                             cudaStream_t stream) {
    VLRF_REQUIRE(n_seqs >= 0 && Hs > 0 && G > 0 && N > 0 && P > 0, "ssd_scan: bad sizes");
    VLRF_REQUIRE(Hs % G == 0, "ssd_scan: %d heads cannot share %d groups", Hs, G);
    VLRF_REQUIRE(N <= 512, "ssd_scan: a state of %d rows is above 512", N);
    VLRF_REQUIRE(channels == Hs * P + 2 * G * N && dt_off + Hs <= ld && (size_t)Hs * N * P <= (size_t)state_row,
                 "ssd_scan: the rows do not hold what the sizes say");
    if (n_seqs == 0) return VLRF_OK;
    // rows a warp: 8 up to 128 rows (many warps hide the latency of a step that has few CTAs), 16 where the step has
    // CTAs enough (a decode step of many sequences, bound by reading and writing the states), more for larger states
    const int PBs = (P + 31) / 32;
    int sms = 0, devi = 0;
    cudaGetDevice(&devi);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, devi);
    const bool many = (long long)Hs * PBs * n_seqs >= 4LL * sms;        // enough CTAs to fill the GPU without many warps each
    const int NR = N > 256 ? 32 : (N > 128 || (many && N >= 64)) ? 16 : N >= 32 ? 8 : 4;
    const int slices = (N + NR - 1) / NR, PB = (P + 31) / 32;
    const bool vec = N % 4 == 0 && (Hs * P) % 4 == 0 && channels % 4 == 0 && (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
    const dim3 grid(Hs * PB, n_seqs), block(slices * 32);
    const int batch = max_new < 1 ? 1 : max_new < SC_MAX_BATCH ? max_new : SC_MAX_BATCH;
    const size_t smem = (size_t)(2 * batch * slices * 32 + 2 * batch * (32 + 2 * ((N + 3) & ~3))) * sizeof(float);
#define GO(R, V) scan_allow_smem<R, V>(smem); launch_chained(ssd_scan_kernel<R, V>, grid, block, smem, stream, xbc, channels, proj, ld, dt_off, dt_bias, a_log, D, state, \
                                state_row, seq_slot, seq_start, seq_pos0, y, Hs, G, N, P, PB, batch)
    if (NR == 4) { if (vec) { GO(4, true); } else { GO(4, false); } }
    else if (NR == 8) { if (vec) { GO(8, true); } else { GO(8, false); } }
    else if (NR == 16) { if (vec) { GO(16, true); } else { GO(16, false); } }
    else { if (vec) { GO(32, true); } else { GO(32, false); } }
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
