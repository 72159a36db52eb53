// Gated linear attention: a recurrent mixer with a matrix of state per head.
//
//   a_t  = sigmoid(z_t + b)^(1/tau)                           one decay per key channel (z_t: a projection of the input)
//   S_t  = diag(a_t) S_{t-1} + k_t v_t^T                      S: [d, dv] float per head and sequence
//   o_t  = S_t^T (q_t * q_scale)
//
// followed, in a second kernel, by an RMS norm of each head's o over dv, a gate silu(g) and the rounding to the
// activation type.  Decays, their logarithms, the state and o are float whatever the projections are stored in.
// The state lives in the cache (one [H, d, dv] block per slot and line): a step loads it, runs its tokens in
// order and writes it back, so a prompt, a prompt that continues and a decode step are the same launch.
#include "common.cuh"

namespace janis {

constexpr int GLA_KS = 16;         // lanes that share a column of the state (each holds a run of DPT key channels)
constexpr int GLA_COLS = 8;        // value columns per CTA

struct GlaRows {
    int row_elems;                 // elements per row of the projected step
    int q_off, k_off, v_off;       // where q [H, d], k [H, d] and v [H, dv] start in a row
    int H, d, dv;
    float q_scale, inv_tau;
};

__device__ __forceinline__ float log_sigmoid(float z) {       // -softplus(-z), stable at both ends
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

// grid (sequences, heads, ceil(dv / GLA_COLS)); 128 threads: thread = (column, ks), ks fastest, so that the 16
// lanes of a column sit in one half of a warp.  Lane ks holds key channels ks * DPT .. ks * DPT + DPT - 1 of its
// column (DPT a multiple of 4, 16 * DPT >= d; channels beyond d hold zeros and decay 1).  A token's q, k and
// decays lie in shared memory as runs of DPT floats, each followed by 4 floats of padding, so that the lanes'
// 16-byte reads fall into different banks.
template <typename T, int DPT>
__global__ void __launch_bounds__(GLA_COLS * GLA_KS)
gla_scan_kernel(const T* __restrict__ rows, GlaRows g, const T* __restrict__ z_rows, const T* __restrict__ z_bias,
                const int* __restrict__ seq_slot, const int* __restrict__ seq_first_row,
                const int* __restrict__ seq_start, const int* __restrict__ seq_end, float* __restrict__ state,
                float* __restrict__ o_out) {
    constexpr int RUN = DPT + 4, TOK = GLA_KS * RUN;       // floats of a lane's run, of a token
    constexpr int GLA_TT = DPT >= 16 ? 8 : 16;             // tokens staged per round (static shared memory stays under 48 KB)
    __shared__ __align__(16) float q_s[GLA_TT * TOK];
    __shared__ __align__(16) float k_s[GLA_TT * TOK];
    __shared__ __align__(16) float a_s[GLA_TT * TOK];
    __shared__ float v_s[GLA_TT * GLA_COLS];
    const int d = g.d, dv = g.dv, H = g.H;
    const int seq = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int tid = threadIdx.x, ks = tid % GLA_KS, col = col0 + tid / GLA_KS;
    const bool live = col < dv;
    grid_dependents_launch();
    const int slot = seq_slot[seq], row0 = seq_first_row[seq], n_tok = seq_end[seq] - seq_start[seq];
    if (n_tok <= 0) return;
    grid_dependency_wait();
    float S[DPT];
    float* st = slot >= 0 ? state + ((size_t)slot * H + h) * d * dv : nullptr;
#pragma unroll
    for (int ii = 0; ii < DPT; ++ii) {
        const int i = ks * DPT + ii;
        S[ii] = (st != nullptr && live && i < d) ? st[(size_t)i * dv + col] : 0.f;
    }
    for (int t0 = 0; t0 < n_tok; t0 += GLA_TT) {
        const int tt_n = min(GLA_TT, n_tok - t0);
        __syncthreads();
        for (int u = tid; u < tt_n * GLA_KS * DPT; u += blockDim.x) {
            const int tt = u / (GLA_KS * DPT), c = u % (GLA_KS * DPT);
            const int at = tt * TOK + (c / DPT) * RUN + c % DPT;
            float q = 0.f, k = 0.f, a = 1.f;
            if (c < d) {
                const T* row = rows + (size_t)(row0 + t0 + tt) * g.row_elems;
                q = to_float(row[g.q_off + h * d + c]) * g.q_scale;
                k = to_float(row[g.k_off + h * d + c]);
                const float z = to_float(z_rows[(size_t)(row0 + t0 + tt) * H * d + h * d + c]) + to_float(z_bias[h * d + c]);
                a = expf(log_sigmoid(z) * g.inv_tau);
            }
            q_s[at] = q;
            k_s[at] = k;
            a_s[at] = a;
        }
        for (int u = tid; u < tt_n * GLA_COLS; u += blockDim.x) {
            const int tt = u / GLA_COLS, c = col0 + u % GLA_COLS;
            v_s[u] = c < dv ? to_float(rows[(size_t)(row0 + t0 + tt) * g.row_elems + g.v_off + h * dv + c]) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < tt_n; ++tt) {
            const float v = v_s[tt * GLA_COLS + tid / GLA_KS];
            const float4* qq = reinterpret_cast<const float4*>(q_s + tt * TOK + ks * RUN);
            const float4* kk = reinterpret_cast<const float4*>(k_s + tt * TOK + ks * RUN);
            const float4* aa = reinterpret_cast<const float4*>(a_s + tt * TOK + ks * RUN);
            float part[4] = {0.f, 0.f, 0.f, 0.f};           // four chains, added in a fixed order
#pragma unroll
            for (int i4 = 0; i4 < DPT / 4; ++i4) {
                const float4 q4 = qq[i4], k4 = kk[i4], a4 = aa[i4];
                S[4 * i4 + 0] = fmaf(a4.x, S[4 * i4 + 0], k4.x * v);
                S[4 * i4 + 1] = fmaf(a4.y, S[4 * i4 + 1], k4.y * v);
                S[4 * i4 + 2] = fmaf(a4.z, S[4 * i4 + 2], k4.z * v);
                S[4 * i4 + 3] = fmaf(a4.w, S[4 * i4 + 3], k4.w * v);
                part[0] = fmaf(S[4 * i4 + 0], q4.x, part[0]);
                part[1] = fmaf(S[4 * i4 + 1], q4.y, part[1]);
                part[2] = fmaf(S[4 * i4 + 2], q4.z, part[2]);
                part[3] = fmaf(S[4 * i4 + 3], q4.w, part[3]);
            }
            float acc = (part[0] + part[1]) + (part[2] + part[3]);
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            if (ks == 0 && live) o_out[(size_t)(row0 + t0 + tt) * H * dv + h * dv + col] = acc;
        }
    }
    if (st != nullptr && live) {
#pragma unroll
        for (int ii = 0; ii < DPT; ++ii) {
            const int i = ks * DPT + ii;
            if (i < d) st[(size_t)i * dv + col] = S[ii];
        }
    }
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :]); a warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ rows, int row_elems, int g_off,
                      const float* __restrict__ w, float eps, T* __restrict__ out, int n_tok, int H, int dv) {
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_dependents_launch();
    grid_dependency_wait();
    if (unit >= n_tok * H) return;
    const int t = unit / H, h = unit % H;
    const float* src = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(src[c], src[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dv + eps);
    const T* gate = rows != nullptr ? rows + (size_t)t * row_elems + g_off + h * dv : nullptr;
    T* dst = out + ((size_t)t * H + h) * dv;
    for (int c = lane; c < dv; c += 32) {
        float y = src[c] * inv * w[c];
        if (gate != nullptr) {
            const float gv = to_float(gate[c]);
            y *= gv / (1.0f + expf(-gv));
        }
        dst[c] = from_float<T>(y);
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT void janis_mixers_set_overlap(int on) { overlap_launches() = on ? 1 : 0; }

JANIS_EXPORT const char* janis_last_error() { return error_buffer(); }

template <typename T>
static int gla_scan_launch(const void* rows, const GlaRows& g, const void* z_rows, const void* z_bias, const int* seq_slot,
                           const int* seq_first_row, const int* seq_start, const int* seq_end, float* state, float* o_out,
                           int n_seq, cudaStream_t stream) {
    const dim3 grid(n_seq, g.H, (g.dv + GLA_COLS - 1) / GLA_COLS), block(GLA_COLS * GLA_KS);
#define JANIS_GLA_CASE(DPT)                                                                                            \
    if (g.d <= GLA_KS * DPT)                                                                                           \
        return launch_kernel("gla_scan", gla_scan_kernel<T, DPT>, grid, block, 0, stream, 1, (const T*)rows, g,        \
                             (const T*)z_rows, (const T*)z_bias, seq_slot, seq_first_row, seq_start, seq_end, state, o_out);
    JANIS_GLA_CASE(4)
    JANIS_GLA_CASE(8)
    JANIS_GLA_CASE(16)
#undef JANIS_GLA_CASE
    return fail("gla_scan: key size %d is above %d", g.d, GLA_KS * 16);
}

JANIS_EXPORT int janis_gla_scan(const void* rows, int dtype, int row_elems, int q_off, int k_off, int v_off,
                                const void* z_rows, const void* z_bias, const int* seq_slot, const int* seq_first_row,
                                const int* seq_start, const int* seq_end, float* state, float* o_out, int n_seq, int H,
                                int d, int dv, float q_scale, float tau, cudaStream_t stream) {
    if (n_seq <= 0) return 0;
    if (H <= 0 || d <= 0 || dv <= 0) return fail("gla_scan: sizes %d heads, %d x %d", H, d, dv);
    if (!(tau > 0.f)) return fail("gla_scan: tau must be positive");
    if (H > 65535) return fail("gla_scan: too many heads (%d)", H);
    GlaRows g;
    g.row_elems = row_elems; g.q_off = q_off; g.k_off = k_off; g.v_off = v_off;
    g.H = H; g.d = d; g.dv = dv; g.q_scale = q_scale; g.inv_tau = 1.0f / tau;
    if (dtype == JANIS_F32)
        return gla_scan_launch<float>(rows, g, z_rows, z_bias, seq_slot, seq_first_row, seq_start, seq_end, state, o_out, n_seq, stream);
    if (dtype == JANIS_BF16)
        return gla_scan_launch<bf16>(rows, g, z_rows, z_bias, seq_slot, seq_first_row, seq_start, seq_end, state, o_out, n_seq, stream);
    return fail("gla_scan: unknown dtype %d", dtype);
}

JANIS_EXPORT int janis_head_norm_gate(const float* o, const void* rows, int dtype, int row_elems, int g_off, const float* w,
                                      float eps, void* out, int T, int H, int dv, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long units = (long long)T * H;
    const dim3 grid((unsigned)((units + 7) / 8)), block(256);
    if (dtype == JANIS_F32)
        return launch_kernel("head_norm_gate", head_norm_gate_kernel<float>, grid, block, 0, stream, 1, o, (const float*)rows,
                             row_elems, g_off, w, eps, (float*)out, T, H, dv);
    if (dtype == JANIS_BF16)
        return launch_kernel("head_norm_gate", head_norm_gate_kernel<bf16>, grid, block, 0, stream, 1, o, (const bf16*)rows,
                             row_elems, g_off, w, eps, (bf16*)out, T, H, dv);
    return fail("gla_scan: unknown dtype %d", dtype);
}
