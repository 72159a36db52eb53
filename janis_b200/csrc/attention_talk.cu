// Attention whose heads talk to each other before the softmax, over the paged cache.
//
//   raw_g[i, j]   = (q_g[i] . k_kv(g)[j]) * scale            for every query head g
//   s_h[i, j]     = sum_g M[h, g] raw_g[i, j]                (M: heads x heads, optional)
//   p_h[i, j]     = exp(s_h[i, j]) / (sink + sum_j' exp(s_h[i, j']))   over the keys j that i sees
//   o_h[i]        = sum_j p_h[i, j] v_kv(h)[j]
//
// A key j is seen by the query at position i when j <= i and, with a block size B > 0, floor(j / B) ==
// floor(i / B).  sink is 1 (a key of score 0 without a value) or 0.  Keys have `d` features and values `dv`,
// which need not be equal.  Values may be stored rotated by their own position (pairs m, m + dv/2, angle
// j * inv_v[m]); the head's output is then turned back by the query's position.
//
// Every kernel here reads keys and values from the cache line only, so a step stores first and attends
// afterwards, and a prompt that continues, a decode step and a layer that reads another layer's line are the
// same launch.  Sizes are run-time numbers.  Scores, weights and sums are float whatever is stored.
#include "common.cuh"

#include <math_constants.h>

namespace janis {

// ---------------------------------------------------------------------------
// Rotary encoding of a step's queries and keys (first `rot` features, pairs i, i + rot/2), rotation of its
// values over all dv features when inv_v is given, and the write of keys and values into the paged cache
// line.  A row of the step holds q (H heads of d), then k (G heads of d), then v (G heads of dv); a layer
// that only reads a line has rows of q alone (with_kv == 0).  One CTA per token.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
qkv_rotate_store_kernel(T* __restrict__ rows, int row_elems, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                        const float* __restrict__ inv_qk, int rot, const float* __restrict__ inv_v, int H, int G, int d,
                        int dv, int with_kv, T* __restrict__ kpool, T* __restrict__ vpool,
                        const int* __restrict__ page_table, int table_stride) {
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x;
    grid_dependents_launch();
    const int pos = tok_pos[t];
    T* kdst = nullptr;
    T* vdst = nullptr;
    if (with_kv) {
        const int slot = seq_slot[tok_seq[t]];
        if (slot >= 0) {
            const int page = page_table[(size_t)slot * table_stride + pos / JANIS_PAGE];
            kdst = kpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * d;
            vdst = vpool + ((size_t)page * G * JANIS_PAGE + pos % JANIS_PAGE) * dv;
        }
    }
    grid_dependency_wait();
    T* row = rows + (size_t)t * row_elems;
    const int hq = rot >> 1, n_rot_heads = with_kv ? H + G : H;
    for (int u = tid; u < n_rot_heads * hq; u += nt) {
        const int head = u / hq, i = u % hq;
        float s, c;
        sincosf((float)pos * inv_qk[i], &s, &c);
        T* p = row + (size_t)head * d;
        float lo, hi;
        rotate_pair(to_float(p[i]), to_float(p[i + hq]), s, c, lo, hi);
        const T tl = from_float<T>(lo), th = from_float<T>(hi);
        p[i] = tl;
        p[i + hq] = th;
        if (head >= H && kdst) {
            T* kd = kdst + (size_t)(head - H) * JANIS_PAGE * d;
            kd[i] = tl;
            kd[i + hq] = th;
        }
    }
    if (!with_kv) return;
    if (kdst && rot < d) {
        const int rest = d - rot;
        for (int u = tid; u < G * rest; u += nt) {
            const int g = u / rest, c = rot + u % rest;
            kdst[(size_t)g * JANIS_PAGE * d + c] = row[(size_t)(H + g) * d + c];
        }
    }
    T* vrow = row + (size_t)(H + G) * d;
    if (inv_v != nullptr) {
        const int hv = dv >> 1;
        for (int u = tid; u < G * hv; u += nt) {
            const int g = u / hv, m = u % hv;
            float s, c;
            sincosf((float)pos * inv_v[m], &s, &c);
            T* p = vrow + (size_t)g * dv;
            float lo, hi;
            rotate_pair(to_float(p[m]), to_float(p[m + hv]), s, c, lo, hi);
            const T tl = from_float<T>(lo), th = from_float<T>(hi);
            p[m] = tl;
            p[m + hv] = th;
            if (vdst) {
                T* vd = vdst + (size_t)g * JANIS_PAGE * dv;
                vd[m] = tl;
                vd[m + hv] = th;
            }
        }
    } else if (vdst) {
        for (int u = tid; u < G * dv; u += nt) vdst[(size_t)(u / dv) * JANIS_PAGE * dv + u % dv] = vrow[u];
    }
}

// ---------------------------------------------------------------------------
// The plain kernel: one CTA per query token, all heads together, tiles of up to 32 keys staged in shared
// memory as floats.  It is the 32-bit path, and the bfloat16 path of sizes the tensor-core kernel leaves out.
// Sums run in an order that depends on the query's position and the model's sizes alone.
// ---------------------------------------------------------------------------
struct TalkShape {
    int H, G, d, dv;
    int block;          // keys are seen within blocks of this many positions (0: all earlier keys)
    int sink;           // 1: one is added to the softmax's denominator
    int kt;             // keys per tile (<= 32)
    float scale;
};

__host__ __device__ inline size_t talk_plain_smem_floats(int H, int G, int d, int dv, int kt) {
    return (size_t)H * d + (size_t)H * H + (size_t)kt * (G * d + 1) + (size_t)kt * G * dv + 2 * (size_t)H * kt +
           (size_t)H * dv + 3 * (size_t)H;
}

template <typename T>
__global__ void __launch_bounds__(256)
talk_attention_plain_kernel(const T* __restrict__ q_rows, int q_row_elems, const int* __restrict__ tok_pos,
                            const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                            const T* __restrict__ kpool, const T* __restrict__ vpool,
                            const int* __restrict__ page_table, int table_stride, const float* __restrict__ talk,
                            const float* __restrict__ inv_v, T* __restrict__ out, TalkShape sh) {
    extern __shared__ float smem[];
    const int H = sh.H, G = sh.G, d = sh.d, dv = sh.dv, KT = sh.kt, rep = H / G;
    const int kstride = G * d + 1;
    float* q_s = smem;
    float* talk_s = q_s + (size_t)H * d;
    float* k_s = talk_s + (size_t)H * H;
    float* v_s = k_s + (size_t)KT * kstride;
    float* raw_s = v_s + (size_t)KT * G * dv;
    float* p_s = raw_s + (size_t)H * KT;
    float* o_s = p_s + (size_t)H * KT;
    float* m_s = o_s + (size_t)H * dv;
    float* l_s = m_s + H;
    float* corr_s = l_s + H;
    const int t = blockIdx.x, tid = threadIdx.x, nt = blockDim.x, lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
    grid_dependents_launch();
    const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
    if (talk != nullptr)
        for (int u = tid; u < H * H; u += nt) talk_s[u] = talk[u];
    grid_dependency_wait();
    T* o_row = out + (size_t)t * H * dv;
    if (slot < 0) {                                   // a padding row: written, never read
        for (int u = tid; u < H * dv; u += nt) o_row[u] = from_float<T>(0.f);
        return;
    }
    const T* q = q_rows + (size_t)t * q_row_elems;
    for (int u = tid; u < H * d; u += nt) q_s[u] = to_float(q[u]);
    for (int u = tid; u < H * dv; u += nt) o_s[u] = 0.f;
    for (int u = tid; u < H; u += nt) {
        m_s[u] = sh.sink ? 0.f : -CUDART_INF_F;
        l_s[u] = sh.sink ? 1.f : 0.f;
    }
    const int first = sh.block > 0 ? (pos / sh.block) * sh.block : 0;
    const int* table = page_table + (size_t)slot * table_stride;
    for (int j0 = first; j0 <= pos; j0 += KT) {
        const int kt = min(KT, pos - j0 + 1);
        __syncthreads();                              // the tile before has been used; q_s and o_s are in place
        for (int u = tid; u < kt * G * d; u += nt) {
            const int jj = u / (G * d), r = u % (G * d), g = r / d, c = r % d, j = j0 + jj;
            const size_t at = (((size_t)table[j / JANIS_PAGE] * G + g) * JANIS_PAGE + j % JANIS_PAGE) * d + c;
            k_s[(size_t)jj * kstride + r] = to_float(kpool[at]);
        }
        for (int u = tid; u < kt * G * dv; u += nt) {
            const int jj = u / (G * dv), r = u % (G * dv), g = r / dv, c = r % dv, j = j0 + jj;
            const size_t at = (((size_t)table[j / JANIS_PAGE] * G + g) * JANIS_PAGE + j % JANIS_PAGE) * dv + c;
            v_s[(size_t)jj * G * dv + r] = to_float(vpool[at]);
        }
        __syncthreads();
        for (int u = tid; u < H * KT; u += nt) {
            const int g = u / KT, jj = u % KT;
            float acc = 0.f;
            if (jj < kt) {
                const float* qq = q_s + (size_t)g * d;
                const float* kk = k_s + (size_t)jj * kstride + (size_t)(g / rep) * d;
                for (int c = 0; c < d; ++c) acc = fmaf(qq[c], kk[c], acc);
            }
            raw_s[u] = acc * sh.scale;
        }
        __syncthreads();
        for (int h = warp; h < H; h += nwarp) {
            float s = -CUDART_INF_F;
            if (lane < kt) {
                if (talk != nullptr) {
                    s = 0.f;
                    for (int g = 0; g < H; ++g) s = fmaf(talk_s[h * H + g], raw_s[g * KT + lane], s);
                } else {
                    s = raw_s[h * KT + lane];
                }
            }
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            const float p = lane < kt ? expf(s - m_new) : 0.f;
            const float sum = warp_sum(p);
            const float corr = m_old == -CUDART_INF_F ? 0.f : expf(m_old - m_new);
            __syncwarp();
            if (lane == 0) {
                l_s[h] = l_s[h] * corr + sum;
                m_s[h] = m_new;
                corr_s[h] = corr;
            }
            if (lane < KT) p_s[h * KT + lane] = p;
        }
        __syncthreads();
        for (int u = tid; u < H * dv; u += nt) {
            const int h = u / dv, c = u % dv;
            const float* vv = v_s + (size_t)(h / rep) * dv + c;
            const float* pp = p_s + h * KT;
            float acc = o_s[u] * corr_s[h];
            for (int jj = 0; jj < kt; ++jj) acc = fmaf(pp[jj], vv[(size_t)jj * G * dv], acc);
            o_s[u] = acc;
        }
    }
    __syncthreads();
    if (inv_v != nullptr) {
        const int hv = dv >> 1;
        for (int u = tid; u < H * hv; u += nt) {
            const int h = u / hv, m = u % hv;
            const float inv_l = 1.f / l_s[h];
            float s, c;
            sincosf((float)pos * inv_v[m], &s, &c);
            float lo, hi;
            rotate_pair(o_s[h * dv + m] * inv_l, o_s[h * dv + m + hv] * inv_l, -s, c, lo, hi);
            o_row[h * dv + m] = from_float<T>(lo);
            o_row[h * dv + m + hv] = from_float<T>(hi);
        }
    } else {
        for (int u = tid; u < H * dv; u += nt) o_row[u] = from_float<T>(o_s[u] / l_s[u / dv]);
    }
}

}  // namespace janis

using namespace janis;

JANIS_EXPORT int janis_qkv_rotate_store(void* rows, int dtype, int row_elems, const int* tok_pos, const int* tok_seq,
                                        const int* seq_slot, const float* inv_qk, int rot, const float* inv_v, int T,
                                        int H, int G, int d, int dv, int with_kv, void* kpool, void* vpool,
                                        const int* page_table, int table_stride, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1)) return fail("qkv_rotate_store: rotary width %d does not fit key size %d", rot, d);
    if (inv_v != nullptr && (dv & 1)) return fail("qkv_rotate_store: rotated values need an even size, found %d", dv);
    if (row_elems < H * d + (with_kv ? G * (d + dv) : 0)) return fail("qkv_rotate_store: rows of %d elements are too short", row_elems);
    if (with_kv && (!kpool || !vpool || !page_table || !seq_slot)) return fail("qkv_rotate_store: no cache line to store into");
    const dim3 grid(T), block(128);
    if (dtype == JANIS_F32)
        return launch_kernel("qkv_rotate_store", qkv_rotate_store_kernel<float>, grid, block, 0, stream, 1, (float*)rows,
                             row_elems, tok_pos, tok_seq, seq_slot, inv_qk, rot, inv_v, H, G, d, dv, with_kv, (float*)kpool,
                             (float*)vpool, page_table, table_stride);
    if (dtype == JANIS_BF16)
        return launch_kernel("qkv_rotate_store", qkv_rotate_store_kernel<bf16>, grid, block, 0, stream, 1, (bf16*)rows,
                             row_elems, tok_pos, tok_seq, seq_slot, inv_qk, rot, inv_v, H, G, d, dv, with_kv, (bf16*)kpool,
                             (bf16*)vpool, page_table, table_stride);
    return fail("qkv_rotate_store: unknown dtype %d", dtype);
}

static int talk_plain_tile(int H, int G, int d, int dv, size_t* bytes) {
    for (int kt = 32; kt >= 1; kt >>= 1) {
        const size_t b = talk_plain_smem_floats(H, G, d, dv, kt) * sizeof(float);
        if (b <= 200 * 1024) {
            *bytes = b;
            return kt;
        }
    }
    return 0;
}

JANIS_EXPORT int janis_talk_attention(const void* q_rows, int dtype, int q_row_elems, const int* tok_pos,
                                      const int* tok_seq, const int* seq_slot, const void* kpool, const void* vpool,
                                      const int* page_table, int table_stride, const float* talk, const float* inv_v,
                                      void* out, int T, int H, int G, int d, int dv, float scale, int block, int sink,
                                      cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G) return fail("talk_attention: %d query heads do not divide over %d key/value heads", H, G);
    if (d <= 0 || dv <= 0) return fail("talk_attention: key size %d, value size %d", d, dv);
    if (inv_v != nullptr && (dv & 1)) return fail("talk_attention: rotated values need an even size, found %d", dv);
    if (q_row_elems < H * d) return fail("talk_attention: query rows of %d elements are too short", q_row_elems);
    if (block < 0) return fail("talk_attention: block size %d", block);
    size_t bytes = 0;
    TalkShape sh;
    sh.H = H; sh.G = G; sh.d = d; sh.dv = dv; sh.block = block; sh.sink = sink ? 1 : 0; sh.scale = scale;
    sh.kt = talk_plain_tile(H, G, d, dv, &bytes);
    if (sh.kt == 0) return fail("talk_attention: heads of these sizes do not fit shared memory (%d x %d, %d x %d)", H, d, G, dv);
    const dim3 grid(T), block_dim(256);
    if (dtype == JANIS_F32) {
        static size_t most_f = 0;
        if (bytes > most_f) {
            cudaError_t e = cudaFuncSetAttribute(talk_attention_plain_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return fail("talk_attention: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e));
            most_f = bytes;
        }
        return launch_kernel("talk_attention", talk_attention_plain_kernel<float>, grid, block_dim, bytes, stream, 1,
                             (const float*)q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, (const float*)kpool,
                             (const float*)vpool, page_table, table_stride, talk, inv_v, (float*)out, sh);
    }
    if (dtype == JANIS_BF16) {
        static size_t most_b = 0;
        if (bytes > most_b) {
            cudaError_t e = cudaFuncSetAttribute(talk_attention_plain_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            if (e != cudaSuccess) return fail("talk_attention: shared memory of %zu bytes refused: %s", bytes, cudaGetErrorString(e));
            most_b = bytes;
        }
        return launch_kernel("talk_attention", talk_attention_plain_kernel<bf16>, grid, block_dim, bytes, stream, 1,
                             (const bf16*)q_rows, q_row_elems, tok_pos, tok_seq, seq_slot, (const bf16*)kpool,
                             (const bf16*)vpool, page_table, table_stride, talk, inv_v, (bf16*)out, sh);
    }
    return fail("talk_attention: unknown dtype %d", dtype);
}
