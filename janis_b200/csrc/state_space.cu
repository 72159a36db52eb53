// State-space mixers: a causal convolution per channel with silu, the selective scan, and the gated norm that
// follows the scan of the state-space-duality form.
//
//   conv:  x'[t, c] = silu(b[c] + sum_j w[c, K-1-j] x[t-j, c])      inputs before the sequence's start are zero;
//          the last K-1 inputs of a sequence are kept per slot, so that a later step goes on from them
//   scan:  S[c, n] <- exp(delta A) S[c, n] + delta u[c] B[n];   o[c] = sum_n S[c, n] C[n] + D u[c]
//          delta = softplus(dt + dt_bias); dt, A's row and D are indexed by c / ch_per_head, B and C by the group
//          c / ch_per_group.  With a state per (channel, n) in A and ch_per_head = 1 this is the selective scan of
//          Mamba; with one number per head in A it is the recurrence of its state-space-duality form.
//   norm:  y = rms_parts(o * silu(z)) * w over equal parts of a row
//
// delta, the decays, the state and o are float whatever the projections are stored in.  The state lives in the
// cache, [slots, C, N] floats per line: a step loads it, runs its tokens in order and writes it back; sequences
// without a slot (padding) start from zero and store nothing.
#include "common.cuh"

namespace janis {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// A state that remembers hundreds of tokens is multiplied by decays just below 1, where a float holds exp(x) to
// 6e-8 only and an error of one sign in every step adds up over the steps.  So the decay is kept as exp(x) - 1, which
// expm1f gives to its own last bit however small it is, and the step is S + (S (exp(x) - 1) + input): the bracket is
// small against S and its rounding does not count; what remains is the one rounding of the sum.
__device__ __forceinline__ float decay_minus_one(float x) { return expm1f(x); }
__device__ __forceinline__ float decayed(float S, float grow, float input) { return S + fmaf(S, grow, input); }

// ---------------------------------------------------------------------------
// convolution: a thread per (token, channel); the taps that reach back before the step come from the slot's state
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const T* __restrict__ rows, int row_elems, int col_off, int C, int K,
                        const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                        const int* __restrict__ seq_first_row, T* __restrict__ out) {
    const int t = blockIdx.x;
    grid_dependents_launch();
    const int s = tok_seq[t], slot = seq_slot[s], i = t - seq_first_row[s];
    grid_dependency_wait();
    const float* st = slot >= 0 ? state + (size_t)slot * max(K - 1, 1) * C : nullptr;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float acc = bias[c];
        const float* wc = w + (size_t)c * K;
        for (int j = 0; j < K; ++j) {
            const int idx = i - j;
            float x = 0.f;
            if (idx >= 0) x = to_float(rows[(size_t)(t - j) * row_elems + col_off + c]);
            else if (st != nullptr) x = st[(size_t)(K - 1 + idx) * C + c];
            acc = fmaf(wc[K - 1 - j], x, acc);
        }
        out[(size_t)t * C + c] = from_float<T>(silu_f(acc));
    }
}

// the K-1 inputs a sequence ends the step with: a thread per (sequence, channel) reads them all, then writes
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T* __restrict__ rows, int row_elems, int col_off, int C, int K, float* __restrict__ state,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                         const int* __restrict__ seq_start, const int* __restrict__ seq_end) {
    const int s = blockIdx.x;
    grid_dependents_launch();
    const int slot = seq_slot[s], row0 = seq_first_row[s], n = seq_end[s] - seq_start[s];
    grid_dependency_wait();
    if (slot < 0 || n <= 0 || K <= 1) return;
    float* st = state + (size_t)slot * (K - 1) * C;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float keep[15];
#pragma unroll
        for (int jj = 0; jj < 15; ++jj) {
            if (jj >= K - 1) break;
            const int idx = n - (K - 1) + jj;
            keep[jj] = idx >= 0 ? to_float(rows[(size_t)(row0 + idx) * row_elems + col_off + c]) : st[(size_t)(jj + n) * C + c];
        }
#pragma unroll
        for (int jj = 0; jj < 15; ++jj) {
            if (jj >= K - 1) break;
            st[(size_t)jj * C + c] = keep[jj];
        }
    }
}

// ---------------------------------------------------------------------------
// scan
// ---------------------------------------------------------------------------
struct ScanShape {
    int u_stride, u_off;           // u[t, c] = u_rows[t * u_stride + u_off + c]
    int dt_stride, dt_off;         // dt[t, c / cph]
    int bc_stride, b_off, c_off;   // B[t, group * N + n], C[t, group * N + n]
    int z_stride, z_off;           // the gate (GATED only)
    int a_per_state;               // A is [C / cph, N] (1) or [C / cph] (0)
    int C, N, cph, cpg;
    int ln;                        // lanes that share a channel (a power of two up to 32); lane l holds states l, l + ln, ...
};

constexpr int SCAN_THREADS = 128;

template <typename T, int SPL, bool GATED>
__global__ void __launch_bounds__(SCAN_THREADS)
selective_scan_kernel(const T* __restrict__ u_rows, const T* __restrict__ dt_rows, const T* __restrict__ bc_rows,
                      const T* __restrict__ z_rows, const float* __restrict__ dt_bias, const float* __restrict__ A,
                      const float* __restrict__ D, ScanShape g, const int* __restrict__ seq_slot,
                      const int* __restrict__ seq_first_row, const int* __restrict__ seq_start,
                      const int* __restrict__ seq_end, float* __restrict__ state, void* __restrict__ out_raw) {
    constexpr int TT = SPL <= 2 ? 8 : (SPL <= 4 ? 4 : 2);          // tokens whose inputs are asked for together
    const int LN = g.ln, N = g.N, C = g.C;
    const int seq = blockIdx.x, tid = threadIdx.x, l = tid & (LN - 1);
    const int c_raw = blockIdx.y * (SCAN_THREADS / LN) + tid / LN;
    const bool live = c_raw < C;
    const int c = live ? c_raw : C - 1;
    const int head = c / g.cph, group = c / g.cpg;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    const float bias = dt_bias[head], Dh = D[head];
    float Areg[SPL];
#pragma unroll
    for (int k = 0; k < SPL; ++k) {
        const int n = l + k * LN;
        Areg[k] = g.a_per_state ? (n < N ? A[(size_t)head * N + n] : 0.f) : A[head];
    }
    grid_dependency_wait();
    float S[SPL];
    float* st = slot >= 0 ? state + ((size_t)slot * C + c) * N : nullptr;
#pragma unroll
    for (int k = 0; k < SPL; ++k) {
        const int n = l + k * LN;
        S[k] = (st != nullptr && n < N) ? st[n] : 0.f;
    }
    const int bcol = g.b_off + group * N, ccol = g.c_off + group * N;
    for (int t0 = 0; t0 < n_tok; t0 += TT) {
        float dtv[TT], uv[TT], zv[TT], Bv[TT][SPL], Cv[TT][SPL];
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            const bool in = t0 + tt < n_tok;
            const size_t row = (size_t)(row0 + t0 + (in ? tt : 0));
            dtv[tt] = to_float(dt_rows[row * g.dt_stride + g.dt_off + head]);
            uv[tt] = to_float(u_rows[row * g.u_stride + g.u_off + c]);
            zv[tt] = GATED ? to_float(z_rows[row * g.z_stride + g.z_off + c]) : 0.f;
#pragma unroll
            for (int k = 0; k < SPL; ++k) {
                const int n = l + k * LN;
                Bv[tt][k] = n < N ? to_float(bc_rows[row * g.bc_stride + bcol + n]) : 0.f;
                Cv[tt][k] = n < N ? to_float(bc_rows[row * g.bc_stride + ccol + n]) : 0.f;
            }
        }
#pragma unroll
        for (int tt = 0; tt < TT; ++tt) {
            if (t0 + tt >= n_tok) break;                       // (uniform over the CTA)
            const float delta = softplus_f(dtv[tt] + bias), du = delta * uv[tt];
            const float x_h = delta * Areg[0];
            const float grow_h = g.a_per_state ? 0.f : decay_minus_one(x_h);
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < SPL; ++k) {
                const float x = g.a_per_state ? delta * Areg[k] : x_h;
                const float grow = g.a_per_state ? decay_minus_one(x) : grow_h;
                S[k] = decayed(S[k], grow, du * Bv[tt][k]);
                acc = fmaf(S[k], Cv[tt][k], acc);
            }
            for (int off = LN >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
            if (l == 0 && live) {
                float y = fmaf(Dh, uv[tt], acc);
                const size_t at = (size_t)(row0 + t0 + tt) * C + c;
                if (GATED) reinterpret_cast<T*>(out_raw)[at] = from_float<T>(y * silu_f(zv[tt]));
                else reinterpret_cast<float*>(out_raw)[at] = y;
            }
        }
    }
    if (st != nullptr && live) {
#pragma unroll
        for (int k = 0; k < SPL; ++k) {
            const int n = l + k * LN;
            if (n < N) st[n] = S[k];
        }
    }
}

// y[t, part] = x / sqrt(mean(x^2) + eps) * w with x = o * silu(z): a CTA per (token, part)
template <typename T>
__global__ void __launch_bounds__(256)
gate_group_norm_kernel(const float* __restrict__ o, const T* __restrict__ rows, int row_elems, int z_off,
                       const float* __restrict__ w, float eps, T* __restrict__ out, int C, int per) {
    __shared__ float scratch[32];
    const int t = blockIdx.x, c0 = blockIdx.y * per;
    grid_dependents_launch();
    grid_dependency_wait();
    const float* src = o + (size_t)t * C + c0;
    const T* z = rows + (size_t)t * row_elems + z_off + c0;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float v = src[i] * silu_f(to_float(z[i]));
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)per + eps);
    T* dst = out + (size_t)t * C + c0;
    for (int i = threadIdx.x; i < per; i += blockDim.x)
        dst[i] = from_float<T>(src[i] * silu_f(to_float(z[i])) * inv * w[c0 + i]);
}

}  // namespace janis

using namespace janis;

template <typename T>
static int conv_launch(const void* rows, int row_elems, int col_off, int C, int K, const float* w, const float* bias,
                       float* state, const int* tok_seq, const int* seq_slot, const int* seq_first_row,
                       const int* seq_start, const int* seq_end, int n_tok, int n_seq, void* out, cudaStream_t stream) {
    const int by = (C + 255) / 256 < 64 ? (C + 255) / 256 : 64;
    if (launch_kernel("causal_conv_silu", causal_conv_silu_kernel<T>, dim3(n_tok, by), dim3(256), 0, stream, 1,
                      (const T*)rows, row_elems, col_off, C, K, w, bias, (const float*)state, tok_seq, seq_slot,
                      seq_first_row, (T*)out))
        return 1;
    if (K <= 1) return 0;
    return launch_kernel("conv_state_update", conv_state_update_kernel<T>, dim3(n_seq, by), dim3(256), 0, stream, 1,
                         (const T*)rows, row_elems, col_off, C, K, state, seq_slot, seq_first_row, seq_start, seq_end);
}

JANIS_EXPORT int janis_causal_conv_silu(const void* rows, int dtype, int row_elems, int col_off, int C, int K,
                                        const float* w, const float* bias, float* state, const int* tok_seq,
                                        const int* seq_slot, const int* seq_first_row, const int* seq_start,
                                        const int* seq_end, int n_tok, int n_seq, void* out, cudaStream_t stream) {
    if (n_tok <= 0 || n_seq <= 0) return 0;
    if (K < 1 || K > 16) return fail("causal_conv_silu: %d taps (1 to 16 are taken)", K);
    if (C <= 0 || col_off < 0 || col_off + C > row_elems) return fail("causal_conv_silu: channels %d at %d do not fit rows of %d", C, col_off, row_elems);
    if (dtype == JANIS_F32)
        return conv_launch<float>(rows, row_elems, col_off, C, K, w, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                                  seq_end, n_tok, n_seq, out, stream);
    if (dtype == JANIS_BF16)
        return conv_launch<bf16>(rows, row_elems, col_off, C, K, w, bias, state, tok_seq, seq_slot, seq_first_row, seq_start,
                                 seq_end, n_tok, n_seq, out, stream);
    return fail("causal_conv_silu: unknown dtype %d", dtype);
}

template <typename T, bool GATED>
static int scan_launch(const void* u, const void* dt, const void* bc, const void* z, const float* dt_bias, const float* A,
                       const float* D, ScanShape g, int spl, const int* seq_slot, const int* seq_first_row,
                       const int* seq_start, const int* seq_end, int n_seq, float* state, void* out, cudaStream_t stream) {
    const int per_cta = SCAN_THREADS / g.ln;
    const dim3 grid(n_seq, (g.C + per_cta - 1) / per_cta), block(SCAN_THREADS);
#define JANIS_SCAN_CASE(SPL)                                                                                           \
    if (spl <= SPL)                                                                                                    \
        return launch_kernel("selective_scan", selective_scan_kernel<T, SPL, GATED>, grid, block, 0, stream, 1,       \
                             (const T*)u, (const T*)dt, (const T*)bc, (const T*)z, dt_bias, A, D, g, seq_slot,          \
                             seq_first_row, seq_start, seq_end, state, out);
    JANIS_SCAN_CASE(1)
    JANIS_SCAN_CASE(2)
    JANIS_SCAN_CASE(3)
    JANIS_SCAN_CASE(4)
    JANIS_SCAN_CASE(6)
    JANIS_SCAN_CASE(8)
    JANIS_SCAN_CASE(16)
#undef JANIS_SCAN_CASE
    return fail("selective_scan: %d states a channel are above %d", g.N, 32 * 16);
}

JANIS_EXPORT int janis_selective_scan(const void* u, int dtype, int u_stride, int u_off, const void* dt, int dt_stride,
                                      int dt_off, const float* dt_bias, const float* A, int a_per_state, const void* bc,
                                      int bc_stride, int b_off, int c_off, const float* D, const void* z, int z_stride,
                                      int z_off, const int* seq_slot, const int* seq_first_row, const int* seq_start,
                                      const int* seq_end, int n_seq, float* state, void* out, int C, int N, int cph,
                                      int cpg, cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    if (C <= 0 || N <= 0 || cph <= 0 || cpg <= 0 || C % cph || C % cpg)
        return fail("selective_scan: %d channels, %d states, %d a head, %d a group", C, N, cph, cpg);
    if (n_seq > 65535 * 32767) return fail("selective_scan: too many sequences (%d)", n_seq);
    ScanShape g;
    g.u_stride = u_stride; g.u_off = u_off; g.dt_stride = dt_stride; g.dt_off = dt_off;
    g.bc_stride = bc_stride; g.b_off = b_off; g.c_off = c_off; g.z_stride = z_stride; g.z_off = z_off;
    g.a_per_state = a_per_state ? 1 : 0; g.C = C; g.N = N; g.cph = cph; g.cpg = cpg;
    // lanes a channel and states a lane: the pair that wastes the fewest places, more lanes on a tie
    static const int spls[7] = {1, 2, 3, 4, 6, 8, 16};
    int best_ln = 0, best_spl = 0, best = 1 << 30;
    for (int ln = 32; ln >= 4; ln >>= 1)
        for (int i = 0; i < 7; ++i)
            if (ln * spls[i] >= N) {
                if (ln * spls[i] < best) { best = ln * spls[i]; best_ln = ln; best_spl = spls[i]; }
                break;
            }
    if (!best_ln) return fail("selective_scan: %d states a channel are above %d", N, 32 * 16);
    g.ln = best_ln;
    const bool gated = z != nullptr;
    if (dtype == JANIS_F32)
        return gated ? scan_launch<float, true>(u, dt, bc, z, dt_bias, A, D, g, best_spl, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream)
                     : scan_launch<float, false>(u, dt, bc, z, dt_bias, A, D, g, best_spl, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream);
    if (dtype == JANIS_BF16)
        return gated ? scan_launch<bf16, true>(u, dt, bc, z, dt_bias, A, D, g, best_spl, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream)
                     : scan_launch<bf16, false>(u, dt, bc, z, dt_bias, A, D, g, best_spl, seq_slot, seq_first_row, seq_start, seq_end, n_seq, state, out, stream);
    return fail("selective_scan: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_gate_group_norm(const float* o, const void* rows, int dtype, int row_elems, int z_off, const float* w,
                                       float eps, int n_groups, void* out, int T, int C, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (n_groups <= 0 || C % n_groups || n_groups > 65535) return fail("gate_group_norm: %d channels in %d parts", C, n_groups);
    const dim3 grid(T, n_groups), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("gate_group_norm", gate_group_norm_kernel<float>, grid, block, 0, stream, 1, o, (const float*)rows,
                             row_elems, z_off, w, eps, (float*)out, C, C / n_groups);
    if (dtype == JANIS_BF16)
        return launch_kernel("gate_group_norm", gate_group_norm_kernel<bf16>, grid, block, 0, stream, 1, o, (const bf16*)rows,
                             row_elems, z_off, w, eps, (bf16*)out, C, C / n_groups);
    return fail("gate_group_norm: unknown dtype %d", dtype);
}
