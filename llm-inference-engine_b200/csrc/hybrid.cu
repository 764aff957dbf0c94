// hybrid.cu -- the layer-list decoder: a model given as a list of layers, each with a token mixer of some kind and an optional
// feed-forward of some kind (b200_hybrid_layer_t), run over a ragged mixed batch of portions (b200_hybrid_batch_t).
//
// One layer = x += rmsnorm(mixer(x)) * g1;  x += rmsnorm(ff(x)) * g2 (B200_NORM_RMS_POST), or x += ls1 * dyt(mixer(dyt(x))); x += ls2 *
// dyt(ff(dyt(x))) (B200_NORM_DYT_PRE_POST: the kernel that adds a sublayer's result also writes the next sublayer's normed input), with x
// the fp32 residual stream.  Launch sequence per layer:
//   fused input projection (b200_linear: tcgen05 GEMM / weight-streaming GEMV by token count)
//   attention mixer:  q/k whole-projection norm + pool append -> chunked sink attention (gate fused) -> output projection
//   gla mixer:        decay (low-rank, fp32) -> recurrence over the state slots -> head norm * silu(gate) -> output projection
//   latent mixer:     split + rotation + latent-row norm + pool append -> grouped GEMM over the heads (q into the latent space) -> windowed
//                     sink attention over the latent rows -> grouped GEMM over the heads (value up-projection) -> gate -> output projection
//   post-norm + residual add (fp32)
//   dense ff:         b200_linear up -> bias + act -> b200_linear down (its bias joins the residual kernel)
//   moe (softmax):    router (fp32) -> route -> plan -> gather rows -> grouped gate|up -> act(gate) * up -> grouped down; shared expert alike;
//                     combine (weights on the outputs, identity experts return the input) + norm + residual add, one kernel
//   moe:              router + shared gate (fp32) -> route -> plan -> gather (weight on the input) -> grouped up (+act) -> grouped down
//                     shared expert: b200_linear up -> act -> b200_linear down
//                     combine (sum of the token's expert rows + gate * shared) + post-norm + residual add, one kernel
// Pre-norm layers on residual streams (B200_NORM_LN_PRE): per sublayer ONE kernel rewrites all streams from the sublayer's result (two
// mixers side by side arrive as two projected rows, each RMS-normed over the width) and leaves the next sublayer's layer-normed input:
//   input projection -> mixer (scored attention | delta rule | state-space | linear attention; a second mixer beside it) -> output
//   projection(s) -> streams + next norm;  gate|up projection -> act(gate) * up -> down projection -> streams + next norm
// and at the end: final norm of the wanted rows -> LM head with fp32 logits (scaled, soft-capped).
// Everything is stream-ordered and allocation-free; the only host->device traffic of a call is one copy of the batch description.
#include "hybrid_ops.cuh"

#include <algorithm>
#include <new>
#include <vector>

namespace b200 {

constexpr int kPageH = B200_KV_PAGE_SIZE;
constexpr int kLatentPartTiles = 1184;     // (one-token tile, key share) pairs the partial-result scratch of the latent attention holds: 148 x 8
constexpr int kLatentHeadsPerTile = 16;  // latent layers with at least this many heads run a decoded token's heads as one tensor-core tile
static size_t align256(size_t v) { return (v + 255) & ~(size_t)255; }

template <typename T>
__global__ void embed_f32_kernel(const int *__restrict__ ids, const T *__restrict__ table, float *__restrict__ x, T *__restrict__ h, int width,
                                 int vocab, float scale) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host has refused ids outside the vocabulary
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = Elem<T>::to_f(table[(size_t)id * width + c]) * scale;
        x[(size_t)t * width + c] = v;
        if (h) h[(size_t)t * width + c] = Elem<T>::from_f(v);  // the 16-bit copy the first projection reads
    }
}

// x[t, :] += rmsnorm(y[t, :]) * g (and h_out[t, :] = T(x[t, :]) for the next projection), where y is either a dense row (y_dense) or the mixture
//   sum_k y_rows[pair_row[t*top + k], :] + shared_gate[t] * y_shared[t, :].   trace (optional) receives the new x.
template <typename T>
__global__ void __launch_bounds__(256)
postnorm_residual_kernel(float *__restrict__ x, const T *__restrict__ y_dense, const T *__restrict__ y_rows, const int *__restrict__ pair_row,
                         int top, const T *__restrict__ y_shared, const float *__restrict__ shared_gate, const float *__restrict__ g, float eps,
                         int width, float *__restrict__ trace, T *__restrict__ h_out) {
    extern __shared__ __align__(16) float ys[];  // [width]
    __shared__ float red[33];
    const int t = blockIdx.x;
    constexpr int V = Elem<T>::kVec;
    // 16-byte pieces when every row starts on a 16-byte boundary (the sums are formed in the same order as element by element)
    const bool vec = width % V == 0 && ((reinterpret_cast<size_t>(x) | reinterpret_cast<size_t>(y_dense) | reinterpret_cast<size_t>(y_rows) |
                                         reinterpret_cast<size_t>(y_shared) | reinterpret_cast<size_t>(g) | reinterpret_cast<size_t>(trace) |
                                         reinterpret_cast<size_t>(h_out)) & 15) == 0;
    float ss = 0.0f;
    if (vec) {
        const float sg = (!y_dense && y_shared) ? shared_gate[t] : 0.0f;
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
            float v[V];
            if (y_dense) {
                unpack16<T>(ld_v4(y_dense + (size_t)t * width + c), v);
            } else {
#pragma unroll
                for (int i = 0; i < V; ++i) v[i] = 0.0f;
                for (int k = 0; k < top; ++k) {
                    float f[V];
                    unpack16<T>(ld_v4(y_rows + (size_t)pair_row[(size_t)t * top + k] * width + c), f);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] += f[i];
                }
                if (y_shared) {
                    float f[V];
                    unpack16<T>(ld_v4(y_shared + (size_t)t * width + c), f);
#pragma unroll
                    for (int i = 0; i < V; ++i) v[i] = fmaf(sg, f[i], v[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < V; i += 4) *reinterpret_cast<float4 *>(ys + c + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
#pragma unroll
            for (int i = 0; i < V; ++i) ss = fmaf(v[i], v[i], ss);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float v;
            if (y_dense) {
                v = Elem<T>::to_f(y_dense[(size_t)t * width + c]);
            } else {
                v = 0.0f;
                for (int k = 0; k < top; ++k) v += Elem<T>::to_f(y_rows[(size_t)pair_row[(size_t)t * top + k] * width + c]);
                if (y_shared) v = fmaf(shared_gate[t], Elem<T>::to_f(y_shared[(size_t)t * width + c]), v);
            }
            ys[c] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    if (vec) {
        for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {  // a thread reads back the pieces of ys it wrote
            float v[V];
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 xv = *reinterpret_cast<const float4 *>(x + (size_t)t * width + c + i);
                const float4 gv = *reinterpret_cast<const float4 *>(g + c + i);
                const float4 yv = *reinterpret_cast<const float4 *>(ys + c + i);
                const float4 r = make_float4(xv.x + yv.x * inv * gv.x, xv.y + yv.y * inv * gv.y, xv.z + yv.z * inv * gv.z, xv.w + yv.w * inv * gv.w);
                *reinterpret_cast<float4 *>(x + (size_t)t * width + c + i) = r;
                if (trace) *reinterpret_cast<float4 *>(trace + (size_t)t * width + c + i) = r;
                v[i] = r.x, v[i + 1] = r.y, v[i + 2] = r.z, v[i + 3] = r.w;
            }
            if (h_out) st_v4(h_out + (size_t)t * width + c, pack16<T>(v));  // what the next sublayer's projections read (16-bit engines)
        }
        return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = x[(size_t)t * width + c] + ys[c] * inv * g[c];
        x[(size_t)t * width + c] = v;
        if (trace) trace[(size_t)t * width + c] = v;
        if (h_out) h_out[(size_t)t * width + c] = Elem<T>::from_f(v);  // what the next sublayer's projections read (16-bit engines)
    }
}

// packed Dynamic-Tanh parameters: [w (width) | b (width) | alpha]
// tanh(z) = sign(z) (1 - 2 / (exp(2|z|) + 1)) in fp32 with the hardware exponential and reciprocal: absolute error of a few 1e-7 over the
// whole range (what fp32 leaves of a value near 1), saturating cleanly; a quarter of the instructions of tanhf, which bounded the kernel
__device__ __forceinline__ float dyt_tanh(float z) {
    const float e = __expf(2.0f * fabsf(z));
    return copysignf(1.0f - __fdividef(2.0f, e + 1.0f), z);
}
__device__ __forceinline__ float dyt_apply(const float *__restrict__ p, int width, int c, float alpha, float v) {
    return fmaf(dyt_tanh(alpha * v), p[c], p[width + c]);
}
// N (a multiple of 4) consecutive elements from column c on, c and width multiples of 4 and p 16-byte aligned: the parameters arrive in
// 16-byte loads (a thread's eight scalar loads of consecutive floats are eight separate cache wavefronts per warp)
template <int N> __device__ __forceinline__ void dyt_apply_vec(const float *__restrict__ p, int width, int c, float alpha, float *v) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 w = *reinterpret_cast<const float4 *>(p + c + i), b = *reinterpret_cast<const float4 *>(p + width + c + i);
        v[i] = fmaf(dyt_tanh(alpha * v[i]), w.x, b.x), v[i + 1] = fmaf(dyt_tanh(alpha * v[i + 1]), w.y, b.y);
        v[i + 2] = fmaf(dyt_tanh(alpha * v[i + 2]), w.z, b.z), v[i + 3] = fmaf(dyt_tanh(alpha * v[i + 3]), w.w, b.w);
    }
}
template <int N> __device__ __forceinline__ void load_vec(const float *__restrict__ p, float *v) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 a = *reinterpret_cast<const float4 *>(p + i);
        v[i] = a.x, v[i + 1] = a.y, v[i + 2] = a.z, v[i + 3] = a.w;
    }
}

// The general form of the kernel above, for either norm kind and either place of the routing weights:
//   y[t, :]  = y_dense[t, :] + y_bias                                                  (a dense sublayer), or
//            = sum_k w(t, k) * (pair_row[t, k] >= 0 ? y_rows[pair_row[t, k], :] : h_in[t, :]) + shared_gate[t] * y_shared[t, :]
//              with w = pair_weight (NULL: 1) and shared_gate NULL: 1; a pair without a row is an identity expert;
//   x[t, :] += ls * norm(y[t, :])    norm = RMS (post = g) or Dynamic Tanh (post packed);   has_y == 0: x stays as it is;
//   h_out[t, :] = T(pre ? dyt(x[t, :]; pre) : x[t, :]): what the next sublayer's projections read.
// h_in and h_out may be the same buffer: an element is read by the thread that overwrites it, before it does.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
sublayer_residual_kernel(float *__restrict__ x, const T *__restrict__ y_dense, const float *__restrict__ y_bias, const T *__restrict__ y_rows,
                         const int *__restrict__ pair_row, const float *__restrict__ pair_weight, int top, const T *__restrict__ y_shared,
                         const float *__restrict__ shared_gate, const T *h_in, int norm, const float *__restrict__ post,
                         const float *__restrict__ ls, float eps, const float *__restrict__ pre, int width, float *__restrict__ trace, T *h_out,
                         int has_y) {
    extern __shared__ __align__(16) float ys[];  // [width]
    __shared__ float red[33];
    constexpr int V = Elem<T>::kVec;
    const int t = blockIdx.x;
    // VEC: 16-byte pieces (every row starts on a 16-byte boundary; the sums are formed in the same order as element by element)
    constexpr bool vec = VEC;
    constexpr int step = VEC ? V : 1;
    const float sg = (has_y && !y_dense && y_shared) ? (shared_gate ? shared_gate[t] : 1.0f) : 0.0f;
    // the sublayer's result for the piece at column c
    auto result = [&](int c, float *v) {
        if (y_dense) {
            if constexpr (vec) unpack16<T>(ld_v4(y_dense + (size_t)t * width + c), v);
            else v[0] = Elem<T>::to_f(y_dense[(size_t)t * width + c]);
            if (y_bias) {
                float b[V];
                if constexpr (vec) load_vec<V>(y_bias + c, b);
                else b[0] = y_bias[c];
                _Pragma("unroll") for (int i = 0; i < step; ++i) v[i] += b[i];
            }
            return;
        }
        _Pragma("unroll") for (int i = 0; i < step; ++i) v[i] = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int r = pair_row[(size_t)t * top + k];
            const float w = pair_weight ? pair_weight[(size_t)t * top + k] : 1.0f;
            const T *src = r >= 0 ? y_rows + (size_t)r * width + c : h_in + (size_t)t * width + c;
            float f[V];
            if constexpr (vec) unpack16<T>(ld_v4(src), f);
            else f[0] = Elem<T>::to_f(src[0]);
            _Pragma("unroll") for (int i = 0; i < step; ++i) v[i] = fmaf(w, f[i], v[i]);
        }
        if (y_shared) {
            float f[V];
            if constexpr (vec) unpack16<T>(ld_v4(y_shared + (size_t)t * width + c), f);
            else f[0] = Elem<T>::to_f(y_shared[(size_t)t * width + c]);
            _Pragma("unroll") for (int i = 0; i < step; ++i) v[i] = fmaf(sg, f[i], v[i]);
        }
    };
    const bool rms = has_y && norm == B200_NORM_RMS_POST;
    float inv = 1.0f;
    if (rms) {  // the mean square needs the whole row first: the row waits in shared memory
        float ss = 0.0f;
        for (int c = threadIdx.x * step; c < width; c += blockDim.x * step) {
            float v[V];
            result(c, v);
            _Pragma("unroll") for (int i = 0; i < step; ++i) {
                ys[c + i] = v[i];
                ss = fmaf(v[i], v[i], ss);
            }
        }
        ss = block_sum(ss, red);
        inv = rsqrtf(ss / (float)width + eps);
    }
    const float a_post = (has_y && !rms) ? post[2 * width] : 0.0f, a_pre = pre ? pre[2 * width] : 0.0f;
    for (int c = threadIdx.x * step; c < width; c += blockDim.x * step) {  // (RMS: a thread reads back the elements of ys it wrote)
        float v[V], y[V];
        if constexpr (vec) {
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 xv = *reinterpret_cast<const float4 *>(x + (size_t)t * width + c + i);
                v[i] = xv.x, v[i + 1] = xv.y, v[i + 2] = xv.z, v[i + 3] = xv.w;
            }
        } else {
            v[0] = x[(size_t)t * width + c];
        }
        if (has_y) {
            float g[V];
            if (rms) {
                if constexpr (vec) load_vec<V>(post + c, g);
                else g[0] = post[c];
                _Pragma("unroll") for (int i = 0; i < step; ++i) y[i] = ys[c + i] * inv * g[i];
            } else {  // Dynamic Tanh works element by element: one pass, nothing staged
                result(c, y);
                if constexpr (vec) dyt_apply_vec<V>(post, width, c, a_post, y);
                else y[0] = dyt_apply(post, width, c, a_post, y[0]);
            }
            if (ls) {
                if constexpr (vec) load_vec<V>(ls + c, g);
                else g[0] = ls[c];
                _Pragma("unroll") for (int i = 0; i < step; ++i) y[i] *= g[i];
            }
            _Pragma("unroll") for (int i = 0; i < step; ++i) v[i] += y[i];
        }
        if constexpr (vec) {
#pragma unroll
            for (int i = 0; i < V; i += 4) {
                const float4 r = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                if (has_y) *reinterpret_cast<float4 *>(x + (size_t)t * width + c + i) = r;
                if (trace) *reinterpret_cast<float4 *>(trace + (size_t)t * width + c + i) = r;
            }
            if (h_out) {
                if (pre) dyt_apply_vec<V>(pre, width, c, a_pre, v);
                st_v4(h_out + (size_t)t * width + c, pack16<T>(v));
            }
        } else {
            if (has_y) x[(size_t)t * width + c] = v[0];
            if (trace) trace[(size_t)t * width + c] = v[0];
            if (h_out) h_out[(size_t)t * width + c] = Elem<T>::from_f(pre ? dyt_apply(pre, width, c, a_pre, v[0]) : v[0]);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
final_dyt_rows_kernel(const float *__restrict__ x, const int *__restrict__ rows, const float *__restrict__ p, float *__restrict__ out,
                      T *__restrict__ out_t, int width) {
    const int i = blockIdx.x;
    const float *xr = x + (size_t)rows[i] * width;
    const float alpha = p[2 * width];
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = dyt_apply(p, width, c, alpha, xr[c]);
        out[(size_t)i * width + c] = v;
        if (out_t) out_t[(size_t)i * width + c] = Elem<T>::from_f(v);
    }
}

__global__ void softcap_kernel(float *__restrict__ logits, size_t n, float scale, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = logits[i] * scale;
        logits[i] = cap > 0.0f ? cap * tanhf(v / cap) : v;
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
final_norm_rows_kernel(const float *__restrict__ x, const int *__restrict__ rows, const float *__restrict__ g, float eps, float *__restrict__ out,
                       T *__restrict__ out_t, int width) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    const float *xr = x + (size_t)rows[i] * width;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = xr[c] * inv * g[c];
        out[(size_t)i * width + c] = v;
        if (out_t) out_t[(size_t)i * width + c] = Elem<T>::from_f(v);
    }
}

// y[m, n] = sum_k x[m, k] w[n, k] (+ bias[n]), fp32 out: used where the result must stay fp32 (router logits, the LM head).
// A CTA stages PM rows of x in shared memory (fp32) and its 8 warps walk the CTA's slice of output columns: a weight row is read once per
// PM activations and the activations once per CTA.
template <typename TX, typename TW, int PM>
__global__ void __launch_bounds__(256)
proj_f32_kernel(const TX *__restrict__ x, int ldx, const TW *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y, int ldy, int M,
                int N, int K, int cols_per_cta) {
    extern __shared__ float xs[];  // [PM][K]
    const int m0 = blockIdx.y * PM, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < PM * K; i += blockDim.x) {
        const int mm = i / K, k = i - mm * K;
        xs[i] = m0 + mm < M ? Elem<TX>::to_f(x[(size_t)(m0 + mm) * ldx + k]) : 0.0f;
    }
    __syncthreads();
    const int n_end = min(N, (int)(blockIdx.x + 1) * cols_per_cta);
    for (int n = blockIdx.x * cols_per_cta + warp; n < n_end; n += 8) {
        float acc[PM] = {};
        const TW *wr = w + (size_t)n * K;
        for (int k = lane; k < K; k += 32) {
            const float wv = Elem<TW>::to_f(wr[k]);
#pragma unroll
            for (int i = 0; i < PM; ++i) acc[i] = fmaf(xs[i * K + k], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < PM; ++i) {
            const float v = warp_sum(acc[i]);
            if (lane == 0 && m0 + i < M) y[(size_t)(m0 + i) * ldy + n] = v + (bias ? bias[n] : 0.0f);
        }
    }
}

// Few outputs (a decode batch's router logits): one warp per output element, four independent partial sums per lane.
template <typename TX, typename TW>
__global__ void __launch_bounds__(256)
proj_f32_small_kernel(const TX *__restrict__ x, int ldx, const TW *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y, int ldy,
                      int M, int N, int K) {
    const int o = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (o >= M * N) return;
    const int mrow = o / N, n = o - mrow * N;
    const TX *xr = x + (size_t)mrow * ldx;
    const TW *wr = w + (size_t)n * K;
    float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
    int k = lane;
    for (; k + 96 < K; k += 128) {
        a0 = fmaf(Elem<TX>::to_f(xr[k]), Elem<TW>::to_f(wr[k]), a0);
        a1 = fmaf(Elem<TX>::to_f(xr[k + 32]), Elem<TW>::to_f(wr[k + 32]), a1);
        a2 = fmaf(Elem<TX>::to_f(xr[k + 64]), Elem<TW>::to_f(wr[k + 64]), a2);
        a3 = fmaf(Elem<TX>::to_f(xr[k + 96]), Elem<TW>::to_f(wr[k + 96]), a3);
    }
    for (; k < K; k += 32) a0 = fmaf(Elem<TX>::to_f(xr[k]), Elem<TW>::to_f(wr[k]), a0);
    const float v = warp_sum((a0 + a1) + (a2 + a3));
    if (lane == 0) y[(size_t)mrow * ldy + n] = v + (bias ? bias[n] : 0.0f);
}

// A decode batch against a wide matrix (M <= 16 rows, any N): one warp per output column walks K in 16-byte pieces; a weight piece is read
// once for all rows, the rows' pieces come from L1 (M * K elements, the same for every warp).  x and w of the same 16-bit type T.
template <typename T, int PM>
__global__ void __launch_bounds__(256)
proj_f32_rows_kernel(const T *__restrict__ x, int ldx, const T *__restrict__ w, const float *__restrict__ bias, float *__restrict__ y, int ldy, int M,
                     int N, int K) {
    constexpr int V = Elem<T>::kVec;
    const int n = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    float acc[PM];
#pragma unroll
    for (int i = 0; i < PM; ++i) acc[i] = 0.0f;
    const T *wr = w + (size_t)n * K;
#pragma unroll 4
    for (int k = lane * V; k < K; k += 32 * V) {
        float wv[V];
        unpack16<T>(ld_stream_v4(wr + k), wv);
#pragma unroll
        for (int i = 0; i < PM; ++i) {
            if (i < M) {
                float xv[V];
                unpack16<T>(ld_v4(x + (size_t)i * ldx + k), xv);
#pragma unroll
                for (int e = 0; e < V; ++e) acc[i] = fmaf(xv[e], wv[e], acc[i]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < PM; ++i) {
        const float v = warp_sum(acc[i]);
        if (lane == 0 && i < M) y[(size_t)i * ldy + n] = v + (bias ? bias[n] : 0.0f);
    }
}

template <typename TX, typename TW, int PM>
static void launch_proj_f32_t(const void *x, int ldx, const void *w, const float *bias, float *y, int ldy, int M, int N, int K, cudaStream_t st) {
    const size_t smem = (size_t)PM * K * sizeof(float);
    // enough CTAs to fill the device, at least 8 columns (one per warp) each
    const int mt = (M + PM - 1) / PM;
    int cols = (N * mt + 4 * 148 - 1) / (4 * 148);
    cols = cols < 8 ? 8 : (cols + 7) / 8 * 8;
    if (smem > 48 * 1024) cudaFuncSetAttribute(proj_f32_kernel<TX, TW, PM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    proj_f32_kernel<TX, TW, PM><<<dim3((N + cols - 1) / cols, mt), 256, smem, st>>>((const TX *)x, ldx, (const TW *)w, bias, y, ldy, M, N, K, cols);
}

int launch_proj_f32(int x_dtype, const void *x, int ldx, int w_dtype, const void *w, const float *bias, float *y, int ldy, int M, int N,
                    int K, cudaStream_t st) {
    if (M == 0) return B200_OK;
    if ((long long)M * N <= 8192) {
        const int grid = (M * N + 7) / 8;
        B200_DISPATCH_DTYPE(w_dtype, {
            if (x_dtype == B200_F32) proj_f32_small_kernel<float, T><<<grid, 256, 0, st>>>((const float *)x, ldx, (const T *)w, bias, y, ldy, M, N, K);
            else proj_f32_small_kernel<T, T><<<grid, 256, 0, st>>>((const T *)x, ldx, (const T *)w, bias, y, ldy, M, N, K);
        });
        return cuda_status("proj_f32 (small) launch");
    }
    if (M <= 16 && x_dtype == w_dtype && w_dtype != B200_F32 && K % 8 == 0 && ldx % 8 == 0 && K >= 512 && aligned16(x) && aligned16(w)) {
        const int grid = (N + 7) / 8;
        if (w_dtype == B200_BF16) {
            if (M <= 8) proj_f32_rows_kernel<__nv_bfloat16, 8><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, ldx, (const __nv_bfloat16 *)w, bias, y, ldy, M, N, K);
            else proj_f32_rows_kernel<__nv_bfloat16, 16><<<grid, 256, 0, st>>>((const __nv_bfloat16 *)x, ldx, (const __nv_bfloat16 *)w, bias, y, ldy, M, N, K);
        } else {
            if (M <= 8) proj_f32_rows_kernel<__half, 8><<<grid, 256, 0, st>>>((const __half *)x, ldx, (const __half *)w, bias, y, ldy, M, N, K);
            else proj_f32_rows_kernel<__half, 16><<<grid, 256, 0, st>>>((const __half *)x, ldx, (const __half *)w, bias, y, ldy, M, N, K);
        }
        return cuda_status("proj_f32 (rows) launch");
    }
    if ((size_t)4 * K * sizeof(float) > 200 * 1024) {
        set_error("proj_f32: K = %d does not fit the shared-memory activation tile", K);
        return B200_ERR_UNSUPPORTED;
    }
    const bool wide = M > 8 && (size_t)16 * K * sizeof(float) <= 200 * 1024, mid = (size_t)8 * K * sizeof(float) <= 200 * 1024;
    B200_DISPATCH_DTYPE(w_dtype, {
        if (x_dtype == B200_F32) {
            if (wide) launch_proj_f32_t<float, T, 16>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else if (mid) launch_proj_f32_t<float, T, 8>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else launch_proj_f32_t<float, T, 4>(x, ldx, w, bias, y, ldy, M, N, K, st);
        } else {
            if (wide) launch_proj_f32_t<T, T, 16>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else if (mid) launch_proj_f32_t<T, T, 8>(x, ldx, w, bias, y, ldy, M, N, K, st);
            else launch_proj_f32_t<T, T, 4>(x, ldx, w, bias, y, ldy, M, N, K, st);
        }
    });
    return cuda_status("proj_f32 launch");
}

// ---- layers of one norm whose sublayers all read it (B200_NORM_LN_PARALLEL)
// x[t, :] = table[id] * scale, and its copy of the engine dtype at h2[t * h2_ld + :] (optional)
template <typename T>
__global__ void embed_rows_kernel(const int *__restrict__ ids, const T *__restrict__ table, float *__restrict__ x, T *__restrict__ h2, int h2_ld,
                                  int width, int vocab, float scale) {
    const int t = blockIdx.x;
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host has refused ids outside the vocabulary
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = Elem<T>::to_f(table[(size_t)id * width + c]) * scale;
        x[(size_t)t * width + c] = v;
        if (h2) h2[(size_t)t * h2_ld + c] = Elem<T>::from_f(v);
    }
}

// The residual step of such a layer and whatever the next layer run reads, in one kernel:
//   v = (replace ? y32[t, :] : x[t, :] + y[t, :]) + bias;   x[t, :] = v;   trace[t, :] = v;
//   h_out[t * h_ld + :] = ln ? T((v - mean) * rsqrt(var + eps) * w + b) : T(v)        (ln packed [w | b]; var = mean of squared deviations)
// y, y32, bias, trace and h_out are optional.  The row waits in shared memory between the passes: mean first, then the deviations.
template <typename T>
__global__ void __launch_bounds__(256)
ln_residual_kernel(float *__restrict__ x, const T *__restrict__ y, const float *__restrict__ y32, const float *__restrict__ bias, int replace,
                   const float *__restrict__ ln, float eps, int width, T *__restrict__ h_out, int h_ld, float *__restrict__ trace) {
    extern __shared__ __align__(16) float row[];  // [width]
    __shared__ float red[33];
    const int t = blockIdx.x;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = replace ? y32[(size_t)t * width + c] : x[(size_t)t * width + c] + (y ? Elem<T>::to_f(y[(size_t)t * width + c]) : 0.0f);
        if (bias) v += bias[c];
        if (replace || y || bias) x[(size_t)t * width + c] = v;
        if (trace) trace[(size_t)t * width + c] = v;
        row[c] = v;
        sum += v;
    }
    if (!h_out) return;
    if (!ln) {
        for (int c = threadIdx.x; c < width; c += blockDim.x) h_out[(size_t)t * h_ld + c] = Elem<T>::from_f(row[c]);  // (a thread reads what it wrote)
        return;
    }
    const float mean = block_sum(sum, red) / (float)width;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row[c] - mean;
        sq = fmaf(d, d, sq);
    }
    const float inv = rsqrtf(block_sum(sq, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) h_out[(size_t)t * h_ld + c] = Elem<T>::from_f(fmaf((row[c] - mean) * inv, ln[c], ln[width + c]));
}

// out[r * out_ld + c] = T(act(in[r * in_ld + gate_col + c]) * in[r * in_ld + up_col + c]): the gated feed-forward's inner row, read from
// and written into rows that other sublayers share.  grid (column blocks, rows); VEC: 16-byte pieces (every piece starts on a 16-byte boundary)
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
gated_act_strided_kernel(const T *__restrict__ in, int in_ld, int gate_col, int up_col, T *__restrict__ out, int out_ld, int inner, int act) {
    constexpr int V = VEC ? Elem<T>::kVec : 1;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (c >= inner) return;
    const T *src = in + (size_t)blockIdx.y * in_ld;
    T *dst = out + (size_t)blockIdx.y * out_ld + c;
    if constexpr (VEC) {
        float g[V], u[V];
        unpack16<T>(ld_v4(src + gate_col + c), g);
        unpack16<T>(ld_v4(src + up_col + c), u);
#pragma unroll
        for (int i = 0; i < V; ++i) g[i] = act_apply(g[i], act) * u[i];
        st_v4(dst, pack16<T>(g));
    } else {
        dst[0] = Elem<T>::from_f(act_apply(Elem<T>::to_f(src[gate_col + c]), act) * Elem<T>::to_f(src[up_col + c]));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
final_ln_rows_kernel(const float *__restrict__ x, const int *__restrict__ rows, const float *__restrict__ p, float eps, float *__restrict__ out,
                     T *__restrict__ out_t, int width) {
    __shared__ float red[33];
    const int i = blockIdx.x;
    const float *xr = x + (size_t)rows[i] * width;
    float sum = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sum += xr[c];
    const float mean = block_sum(sum, red) / (float)width;
    float sq = 0.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) sq = fmaf(xr[c] - mean, xr[c] - mean, sq);
    const float inv = rsqrtf(block_sum(sq, red) / (float)width + eps);
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = fmaf((xr[c] - mean) * inv, p[c], p[width + c]);
        out[(size_t)i * width + c] = v;
        if (out_t) out_t[(size_t)i * width + c] = Elem<T>::from_f(v);
    }
}

// ---- pre-norm layers on residual streams (B200_NORM_LN_PRE)
// One sublayer's residual step on S streams xs [tokens, S, width] and whatever the next sublayer reads, in one kernel:
//   y[t, :]   = ya[t, :]                                                     (one projected row), or
//             = sa * rmsnorm(ya[t, :]) * na + sb * rmsnorm(yb[t, :]) * nb       (two mixers side by side, each normed over the width);
//   xs[t, v]  = sum_s mix[s][v] * xs[t, s] + out[v] * y[t, :]   for all v at once (hc packed [in | out | mix]; NULL: xs += y), or, with
//               x_init, every stream = x_init[t, :] (the embedding output; no y);
//   sum_out / trace [t, :] = sum_v xs[t, v];
//   h_out[t, :] = T(layernorm(sum_v in_next[v] * xs[t, v]; ln_next))              (hc_next packed alike; NULL: the one stream itself).
// Everything is fp32; the row waits in shared memory between the passes (mean first, then the squared deviations).
constexpr int kMaxStreams = 8;
// SC: the stream count at compile time (0: any count up to kMaxStreams, given as S).  VEC: four columns per access.  The coefficients live
// in registers; a thread's loads of one piece (all streams and both rows) are independent of one another and in flight together.
template <typename T, int SC, bool VEC>
__global__ void __launch_bounds__(256)
stream_residual_kernel(float *xs, int S_any, const float *__restrict__ x_init, const T *__restrict__ ya, const T *__restrict__ yb,
                       const float *__restrict__ na, const float *__restrict__ nb, float sa, float sb, const float *__restrict__ hc,
                       const float *__restrict__ hc_next, const float *__restrict__ ln_next, float eps, int width, T *__restrict__ h_out,
                       float *__restrict__ sum_out, float *__restrict__ trace) {
    extern __shared__ __align__(16) float row[];  // [width]
    __shared__ float red[33];
    constexpr int N = VEC ? 4 : 1, SM = SC > 0 ? SC : kMaxStreams;
    const int S = SC > 0 ? SC : S_any;
    const int t = blockIdx.x;
    float c_out[SM], c_in[SM], c_mix[SM][SM];  // c_mix[from][to]
#pragma unroll
    for (int v = 0; v < SM; ++v) {
        c_out[v] = (v < S && hc) ? hc[S + v] : 1.0f;
        c_in[v] = (v < S && hc_next) ? hc_next[v] : 1.0f;
#pragma unroll
        for (int q = 0; q < SM; ++q) c_mix[q][v] = (v < S && q < S && hc) ? hc[2 * S + q * S + v] : (q == v ? 1.0f : 0.0f);
    }
    const T *yar = ya + (size_t)t * width, *ybr = yb + (size_t)t * width;
    float ia = 1.0f, ib = 1.0f;
    if (ya && na) {  // (uniform over the CTA)
        float ssa = 0.0f, ssb = 0.0f;
        for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
            float a[N], b[N];
            load_n<T, N>(yar + c, a);
#pragma unroll
            for (int i = 0; i < N; ++i) ssa = fmaf(a[i], a[i], ssa);
            if (yb) {
                load_n<T, N>(ybr + c, b);
#pragma unroll
                for (int i = 0; i < N; ++i) ssb = fmaf(b[i], b[i], ssb);
            }
        }
        ia = sa * rsqrtf(block_sum(ssa, red) / (float)width + eps);
        if (yb) ib = sb * rsqrtf(block_sum(ssb, red) / (float)width + eps);
    }
    float sum = 0.0f;
    for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
        float y[N], old[SM][N];
#pragma unroll
        for (int v = 0; v < SM; ++v)
            if (v < S) load_n<float, N>(x_init ? x_init + (size_t)t * width + c : xs + ((size_t)t * S + v) * width + c, old[v]);
#pragma unroll
        for (int i = 0; i < N; ++i) y[i] = 0.0f;
        if (ya) {
            load_n<T, N>(yar + c, y);
            if (na) {
                float w[N];
                load_n<float, N>(na + c, w);
#pragma unroll
                for (int i = 0; i < N; ++i) y[i] *= ia * w[i];
                if (yb) {
                    float b[N];
                    load_n<T, N>(ybr + c, b);
                    load_n<float, N>(nb + c, w);
#pragma unroll
                    for (int i = 0; i < N; ++i) y[i] = fmaf(b[i] * ib, w[i], y[i]);
                }
            }
        }
        float u[N], total[N];
#pragma unroll
        for (int i = 0; i < N; ++i) u[i] = total[i] = 0.0f;
#pragma unroll
        for (int v = 0; v < SM; ++v) {
            if (v < S) {
                float a[N];
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    if (x_init) {
                        a[i] = old[v][i];
                    } else {
                        a[i] = c_out[v] * y[i];
#pragma unroll
                        for (int q = 0; q < SM; ++q)
                            if (q < S) a[i] = fmaf(c_mix[q][v], old[q][i], a[i]);
                    }
                    total[i] += a[i];
                    u[i] = fmaf(c_in[v], a[i], u[i]);
                }
                if (x_init || ya) store_n<float, N>(xs + ((size_t)t * S + v) * width + c, a);
            }
        }
        if (trace) store_n<float, N>(trace + (size_t)t * width + c, total);
        if (sum_out) store_n<float, N>(sum_out + (size_t)t * width + c, total);
#pragma unroll
        for (int i = 0; i < N; ++i) row[c + i] = u[i], sum += u[i];
    }
    if (!h_out) return;
    const float mean = block_sum(sum, red) / (float)width;
    float sq = 0.0f;
    for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {  // (a thread reads back the pieces of row[] it wrote)
#pragma unroll
        for (int i = 0; i < N; ++i) {
            const float dv = row[c + i] - mean;
            sq = fmaf(dv, dv, sq);
        }
    }
    const float inv = rsqrtf(block_sum(sq, red) / (float)width + eps);
    for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
        float w[N], b[N], o[N];
        load_n<float, N>(ln_next + c, w);
        load_n<float, N>(ln_next + width + c, b);
#pragma unroll
        for (int i = 0; i < N; ++i) o[i] = fmaf((row[c + i] - mean) * inv, w[i], b[i]);
        store_n<T, N>(h_out + (size_t)t * width + c, o);
    }
}

// where one mixer of one layer run keeps what it remembers
struct MixerPlan {
    size_t k_off = 0, v_off = 0;      // attention kinds: byte offsets into the kv pool (set by set_pools); LATENT: k_off of the rows it reads
    size_t state_off = 0;             // recurrent kinds: byte offset of the matrix state in the state pool
    size_t aux_off = 0, aux2_off = 0; // DELTA: the convolutions' inputs;  MLSTM: the normaliser and the running maximum
};
struct LayerPlan : MixerPlan {
    int n_in = 0;                     // rows of the fused input projection
    int layer = 0;                    // which layer this run executes
    int entry = -1;                   // >= 0: the run opens pass `entry` of the looped block (the entry step comes first)
    MixerPlan side;                   // the second mixer beside the first
};

}  // namespace b200

using namespace b200;

struct b200_hybrid {
    b200_hybrid_config_t cfg;
    std::vector<b200_hybrid_layer_t> layers;
    std::vector<char> layer_set;
    std::vector<LayerPlan> plan;                // one per layer RUN (a looped layer runs several times, each with a cache of its own)
    std::vector<b200_hybrid_layer_t> sides;     // the engine's copies of the second mixers (layers[i].side points here)
    const void *embedding = nullptr, *lm_head = nullptr, *w_entry = nullptr;
    const float *final_norm = nullptr, *loop_step = nullptr;
    char *kv_pool = nullptr, *state_pool = nullptr;
    int num_pages = 0, num_slots = 0;
    // scratch carve-up
    char *scratch = nullptr;
    float *x = nullptr, *f32a = nullptr, *f32b = nullptr, *xn = nullptr;
    void *h = nullptr, *proj = nullptr, *mix = nullptr, *mix2 = nullptr, *y = nullptr, *xg = nullptr, *u = nullptr, *yrows = nullptr, *us = nullptr,
         *ys = nullptr, *lqn = nullptr, *lqr = nullptr, *lql = nullptr, *lol = nullptr, *lov = nullptr;
    float *lpart = nullptr, *rec = nullptr, *f32c = nullptr, *xs = nullptr;
    void *cat = nullptr, *xc = nullptr;
    int *meta = nullptr, *moe_i = nullptr;
    float *moe_f = nullptr;
    std::vector<int> host_meta;
};

namespace {

struct Carve {
    size_t x, f32a, f32b, xn, h, proj, mix, y, xg, u, yrows, us, ys, lqn, lqr, lql, lov, lpart, meta, moe_i, moe_f, rec, f32c, cat, xc, xs, total;
};

// rows of the input projection and columns of the output projection that ONE mixer owns
int mixer_rows(const b200_hybrid_layer_t &l) {
    if (l.mixer == B200_MIXER_ATTN_SCORED) return (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim + (l.out_gate ? l.heads * l.vdim : 0);
    if (l.mixer == B200_MIXER_DELTA)
        return 2 * l.kv_heads * l.dim + l.heads * l.vdim + l.heads + (l.decay_rank > 0 ? l.decay_rank + l.gate_rank : l.heads + l.heads * l.vdim);
    if (l.mixer == B200_MIXER_MLSTM) return 2 * l.heads * l.dim + 2 * l.heads * l.vdim + 2 * l.heads;
    if (l.mixer == B200_MIXER_SSD) return 2 * l.heads * l.vdim + 2 * l.kv_heads * l.dim + l.heads;
    if (l.mixer == B200_MIXER_LINEAR) return 2 * l.heads * l.dim + 2 * l.heads * l.vdim;
    return 0;
}
// channels of the short convolution whose last inputs are part of the state
int conv_channels(const b200_hybrid_layer_t &l) {
    if (l.mixer == B200_MIXER_DELTA) return 2 * l.kv_heads * l.dim + l.heads * l.vdim;
    if (l.mixer == B200_MIXER_SSD) return l.heads * l.vdim + 2 * l.kv_heads * l.dim;
    return 0;
}
int cat_cols(const b200_hybrid_layer_t &l) {
    return l.heads * l.vdim + (l.side ? l.side->heads * l.side->vdim : 0) + (l.mlp == B200_MLP_DENSE ? l.expert_ff : 0);
}
int rec_cols(const b200_hybrid_layer_t &l) {
    if (l.mixer == B200_MIXER_DELTA) return delta_row(l.heads, l.kv_heads, l.dim, l.vdim).ld;
    if (l.mixer == B200_MIXER_MLSTM) return mlstm_row(l.heads, l.dim, l.vdim).ld;
    if (l.mixer == B200_MIXER_SSD) return decay_row(l.heads, l.kv_heads, l.dim, l.vdim).ld;
    if (l.mixer == B200_MIXER_LINEAR) return decay_row(l.heads, l.heads, l.dim, l.vdim).ld;
    return 0;
}

int max_rows_of(const b200_hybrid_config_t &c, const b200_hybrid_layer_t &l) {
    const int pairs = c.max_tokens * l.top;
    return ((pairs + 127) / 128 + l.experts) * 128;  // the larger of the two row-tile sizes
}

int n_in_of(const b200_hybrid_layer_t &l) {
    if (l.norm == B200_NORM_LN_PARALLEL) return mixer_rows(l) + (l.side ? mixer_rows(*l.side) : 0) + (l.mlp == B200_MLP_DENSE ? 2 * l.expert_ff : 0);
    if (l.norm == B200_NORM_LN_PRE) return mixer_rows(l) + (l.side ? mixer_rows(*l.side) : 0);
    if (l.mixer == B200_MIXER_ATTN_CHUNKED) return (2 * l.heads + l.kv_heads) * l.dim;
    if (l.mixer == B200_MIXER_LATENT) return l.heads * (l.dim + l.rot_dim) + l.heads * l.vdim + (l.kv_from < 0 ? l.kv_rank + l.rot_dim : 0);
    return 2 * l.heads * l.dim + 2 * l.heads * l.vdim + l.decay_rank;
}

Carve carve(const b200_hybrid *m) {
    const b200_hybrid_config_t &c = m->cfg;
    const size_t T = (size_t)c.max_tokens, es = c.dtype == B200_F32 ? 4 : 2;
    size_t n_in = 1, n_mix = 1, n_f32 = 1, rows = 0, ff = 1, sff = 1, experts = 1, top = 1, lqn = 0, lqr = 0, lql = 0, lov = 0, lheads = 0, lpart = 0;
    size_t n_rec = 0, n_heads = 0, n_cat = 0;
    bool pre_norm = false;
    const size_t t_pad = (T + 127) / 128 * 128;  // rows per head of the latent mixer's grouped GEMMs
    for (int i = 0; i < c.num_layers; ++i) {
        if (!m->layer_set[i]) continue;
        const b200_hybrid_layer_t &l = m->layers[i];
        n_in = std::max(n_in, (size_t)n_in_of(l));
        n_mix = std::max(n_mix, (size_t)l.heads * std::max(l.dim, l.vdim));
        n_f32 = std::max(n_f32, (size_t)l.heads * std::max(l.dim, l.vdim));
        n_mix = std::max(n_mix, (size_t)l.heads * l.vdim);
        if (l.norm == B200_NORM_LN_PARALLEL || l.norm == B200_NORM_LN_PRE) {
            if (l.norm == B200_NORM_LN_PARALLEL) n_cat = std::max(n_cat, (size_t)cat_cols(l));
            else n_cat = std::max(n_cat, (size_t)l.heads * l.vdim), sff = std::max(sff, (size_t)3 * l.expert_ff), pre_norm = true;
            for (const b200_hybrid_layer_t *mx : {&l, l.side}) {
                if (!mx) continue;
                n_mix = std::max(n_mix, (size_t)mx->heads * std::max(mx->dim, mx->vdim));
                n_mix = std::max(n_mix, (size_t)mx->decay_rank + mx->gate_rank + 256);  // the delta rule's two low-rank inputs as dense rows
                n_f32 = std::max(n_f32, (size_t)mx->heads * std::max(mx->dim, mx->vdim));
                n_rec = std::max(n_rec, (size_t)rec_cols(*mx)), n_heads = std::max(n_heads, (size_t)mx->heads);
            }
            continue;
        }
        if (l.mixer == B200_MIXER_LATENT) {
            lqn = std::max(lqn, (size_t)l.heads * t_pad * l.dim), lqr = std::max(lqr, T * l.heads * l.rot_dim);
            lql = std::max(lql, (size_t)l.heads * t_pad * l.kv_rank), lov = std::max(lov, (size_t)l.heads * t_pad * l.vdim);
            lheads = std::max(lheads, (size_t)l.heads);
            lpart = std::max(lpart, (size_t)kLatentPartTiles * l.heads * (l.kv_rank + 2));
        }
        const size_t g = l.gated ? 3 : 1;  // gated: [gate | up] and the product beside it
        if (l.mlp == B200_MLP_MOE) {
            rows = std::max(rows, (size_t)max_rows_of(c, l));
            ff = std::max(ff, g * l.expert_ff), sff = std::max(sff, g * l.shared_ff);
            experts = std::max(experts, (size_t)l.experts), top = std::max(top, (size_t)l.top);
            n_f32 = std::max(n_f32, (size_t)l.experts + std::max(1, l.identity));
        } else if (l.mlp == B200_MLP_DENSE) {
            sff = std::max(sff, g * l.expert_ff);
        }
    }
    Carve k;
    k.x = align256(T * c.width * 4);
    k.f32a = align256(T * n_f32 * 4);
    k.f32b = align256(T * n_f32 * 4);
    k.xn = align256(T * c.width * 4);
    k.h = align256(T * c.width * es);
    k.proj = align256(T * n_in * es);
    k.mix = align256(T * n_mix * es);
    k.y = align256(T * c.width * es);
    k.xg = align256(rows * c.width * es);
    k.u = align256(rows * ff * es);
    k.yrows = align256(rows * c.width * es);
    k.us = align256(T * sff * es);
    k.ys = align256(T * c.width * es);
    k.lqn = align256(lqn * es), k.lqr = align256(lqr * es), k.lql = align256(lql * es), k.lov = align256(lov * es);
    k.lpart = align256(lpart * 4);
    // meta: attention tiles [4 * (T/64 + S), padded] | ids | tok_seq | tok_pos | want | short-portion token list [T each] | seq_start [S+1] |
    //       pos0 | slot [S each] | block table [S * mpps]
    //       | latent mixers: one-token tiles of the short portions [4 * T] | head of every row tile of 64 and of 128 [heads * t_pad / 64,
    //         heads * t_pad / 128] | live row tiles per layer, of 64 and of 128 [layers each]
    k.meta = align256((4 * (T / 64 + (size_t)c.max_seqs + 1) + 5 * T + 3 * (size_t)c.max_seqs + 1 + (size_t)c.max_seqs * c.max_pages_per_seq +
                       (lheads ? 4 * T : 0) + 2 * lheads * (t_pad / 64) + 2 * (size_t)c.num_layers) * 4);
    // moe ints: sel_expert | pair_row [T*top each] | row_token [rows] | tile_expert [rows / tile] | n_tiles
    k.moe_i = align256((2 * T * top + rows + rows / kMoeTileM + 4) * 4);
    // moe floats: sel_weight [T*top] | row_weight [rows] | shared_gate [T]
    k.moe_f = align256((T * top + rows + T) * 4);
    k.rec = align256(T * n_rec * 4), k.f32c = align256(2 * T * n_heads * 4), k.cat = align256(T * n_cat * es);
    k.xc = (c.loop_times > 0 && !pre_norm) ? align256(2 * T * c.width * es) : 0;
    k.xs = pre_norm ? align256(T * (size_t)std::max(c.streams, 1) * c.width * 4) : 0;
    k.total = k.xs + k.x + k.f32a + k.f32b + k.xn + k.h + k.proj + 2 * k.mix + k.y + k.xg + k.u + k.yrows + k.us + k.ys + k.lqn + k.lqr + 2 * k.lql +
              k.lov + k.lpart + k.meta + k.moe_i + k.moe_f + k.rec + k.f32c + k.cat + k.xc;
    return k;
}

int linear(const b200_hybrid *m, const void *x, const void *w, void *y, int M, int K, int N, cudaStream_t st) {
    return b200_linear(x, w, nullptr, nullptr, y, M, K, N, m->cfg.dtype, B200_W_DENSE, B200_LAYOUT_NK, 0, (b200_stream_t)st);
}

}  // namespace

extern "C" {

b200_hybrid_t *b200_hybrid_create(const b200_hybrid_config_t *cfg) {
    if (!cfg || cfg->width <= 0 || cfg->vocab <= 0 || cfg->num_layers <= 0 || cfg->max_tokens <= 0 || cfg->max_seqs <= 0 ||
        cfg->max_pages_per_seq <= 0 || (cfg->dtype != B200_F32 && cfg->dtype != B200_F16 && cfg->dtype != B200_BF16)) {
        set_error("hybrid_create: bad configuration");
        return nullptr;
    }
    if (cfg->streams < 0 || cfg->streams > kMaxStreams) {
        set_error("hybrid_create: %d residual streams outside [1, %d]", cfg->streams, kMaxStreams);
        return nullptr;
    }
    b200_hybrid *m = new (std::nothrow) b200_hybrid();
    if (!m) return nullptr;
    m->cfg = *cfg;
    m->layers.resize(cfg->num_layers);
    m->sides.resize(cfg->num_layers);
    m->layer_set.assign(cfg->num_layers, 0);
    if (cfg->loop_times > 0) {
        if (cfg->loop_start < 0 || cfg->loop_stop <= cfg->loop_start || cfg->loop_stop > cfg->num_layers) {
            set_error("hybrid_create: looped block [%d, %d) outside the %d layers", cfg->loop_start, cfg->loop_stop, cfg->num_layers);
            delete m;
            return nullptr;
        }
        for (int i = 0; i < cfg->loop_start; ++i) m->plan.push_back(LayerPlan()), m->plan.back().layer = i;
        for (int t = 0; t < cfg->loop_times; ++t)
            for (int i = cfg->loop_start; i < cfg->loop_stop; ++i) {
                m->plan.push_back(LayerPlan());
                m->plan.back().layer = i, m->plan.back().entry = i == cfg->loop_start ? t : -1;
            }
        for (int i = cfg->loop_stop; i < cfg->num_layers; ++i) m->plan.push_back(LayerPlan()), m->plan.back().layer = i;
    } else {
        m->plan.resize(cfg->num_layers);
        for (int i = 0; i < cfg->num_layers; ++i) m->plan[i].layer = i;
    }
    return m;
}

void b200_hybrid_destroy(b200_hybrid_t *m) { delete m; }

static int check_scored_mixer(const b200_hybrid_layer_t *w) {
    B200_REQUIRE(w->heads > 0 && w->dim > 0 && w->vdim > 0, "hybrid_set_layer: mixer sizes missing");
    if (w->mixer == B200_MIXER_ATTN_SCORED) {
        B200_REQUIRE(w->kv_heads > 0 && w->heads % w->kv_heads == 0, "hybrid_set_layer: heads %d not a multiple of kv_heads %d", w->heads, w->kv_heads);
        B200_REQUIRE(w->rot_dims >= 0 && w->rot_dims <= w->dim && w->rot_dims % 2 == 0 && (w->rot_dims == 0 || w->rot_base > 0.0f),
                     "hybrid_set_layer: %d rotating dimensions do not fit a head of %d (even, with a positive base)", w->rot_dims, w->dim);
        B200_REQUIRE(w->window >= 0 && (w->attn_weight == B200_ATTN_SOFTMAX || w->attn_weight == B200_ATTN_SIGMOID), "hybrid_set_layer: bad window or weight kind");
        B200_REQUIRE((w->dist_r1 == nullptr) == (w->dist_r2 == nullptr), "hybrid_set_layer: the distance penalty needs both of its vectors");
        B200_REQUIRE((w->q_norm == nullptr) == (w->k_norm == nullptr), "hybrid_set_layer: q and k are normed together or not at all");
    } else if (w->mixer == B200_MIXER_DELTA) {
        B200_REQUIRE(w->kv_heads > 0 && w->heads % w->kv_heads == 0, "hybrid_set_layer: heads %d not a multiple of kv_heads %d", w->heads, w->kv_heads);
        B200_REQUIRE(w->conv >= 1 && w->conv <= 64 && w->conv_w && w->a_log && w->out_norm && w->decay_rank >= 0, "hybrid_set_layer: delta-rule sizes / weights missing");
        if (w->decay_rank > 0) B200_REQUIRE(w->gate_rank > 0 && w->w_decay && w->w_gate2, "hybrid_set_layer: the delta rule's low-rank halves are missing");
    } else if (w->mixer == B200_MIXER_MLSTM) {
        B200_REQUIRE(w->out_norm && w->gate_cap >= 0.0f, "hybrid_set_layer: matrix-memory weights missing");
    } else if (w->mixer == B200_MIXER_SSD) {
        B200_REQUIRE(w->kv_heads > 0 && w->heads % w->kv_heads == 0, "hybrid_set_layer: heads %d not a multiple of the %d groups", w->heads, w->kv_heads);
        B200_REQUIRE(w->conv >= 1 && w->conv <= 64 && w->conv_w && w->a_log && w->out_norm, "hybrid_set_layer: state-space sizes / weights missing");
        B200_REQUIRE(w->norm_groups >= 1 && (w->heads * w->vdim) % w->norm_groups == 0, "hybrid_set_layer: %d norm groups do not divide %d channels",
                     w->norm_groups, w->heads * w->vdim);
    } else if (w->mixer == B200_MIXER_LINEAR) {
        B200_REQUIRE(w->head_decay && w->out_norm, "hybrid_set_layer: linear-attention weights missing");
    } else {
        set_error("hybrid_set_layer: mixer kind %d cannot share a norm with the feed-forward", w->mixer);
        return B200_ERR_INVALID_ARG;
    }
    return B200_OK;
}

int b200_hybrid_set_layer(b200_hybrid_t *m, int layer, const b200_hybrid_layer_t *w) {
    B200_REQUIRE(m && w, "hybrid_set_layer: null argument");
    B200_REQUIRE(layer >= 0 && layer < m->cfg.num_layers, "hybrid_set_layer: layer %d outside [0, %d)", layer, m->cfg.num_layers);
    B200_REQUIRE(w->mixer >= B200_MIXER_ATTN_CHUNKED && w->mixer <= B200_MIXER_LINEAR, "hybrid_set_layer: unknown mixer kind %d", w->mixer);
    B200_REQUIRE(w->norm >= B200_NORM_RMS_POST && w->norm <= B200_NORM_LN_PRE, "hybrid_set_layer: unknown norm kind %d", w->norm);
    B200_REQUIRE(w->heads > 0 && w->dim > 0 && w->w_in && w->w_out, "hybrid_set_layer: mixer sizes / weights missing");
    if (w->norm == B200_NORM_LN_PARALLEL || w->norm == B200_NORM_LN_PRE) {
        // LN_PARALLEL: one norm, one input projection, one output projection; the mixers are of the kinds that read a shared projection
        const bool pre = w->norm == B200_NORM_LN_PRE;
        B200_REQUIRE(w->pre1, "hybrid_set_layer: norm parameters missing");
        int rc = check_scored_mixer(w);
        if (rc != B200_OK) return rc;
        if (!pre) B200_REQUIRE(w->mixer != B200_MIXER_SSD && w->mixer != B200_MIXER_LINEAR, "hybrid_set_layer: mixer kind %d needs the pre-norm layer form", w->mixer);
        if (w->side) {
            B200_REQUIRE(!w->side->side, "hybrid_set_layer: a second mixer has no second mixer of its own");
            if ((rc = check_scored_mixer(w->side)) != B200_OK) return rc;
            if (pre) B200_REQUIRE(w->side->w_out && (w->branch_norm == nullptr) == (w->side->branch_norm == nullptr),
                                  "hybrid_set_layer: the second mixer needs its output projection, and both mixers a norm of their results or neither");
        }
        B200_REQUIRE(w->mlp == B200_MLP_NONE || (w->mlp == B200_MLP_DENSE && w->gated && w->expert_ff > 0),
                     "hybrid_set_layer: the feed-forward of this layer form is a gated dense one or none");
        if (pre) {
            B200_REQUIRE(w->mlp == B200_MLP_NONE || (w->pre2 && w->w_up && w->w_down), "hybrid_set_layer: feed-forward norm / weights missing");
            B200_REQUIRE(std::max(m->cfg.streams, 1) == 1 || (w->hc1 && (w->mlp == B200_MLP_NONE || w->hc2)), "hybrid_set_layer: stream coefficients missing");
        }
        B200_REQUIRE(w->act >= B200_ACT_RELU2 && w->act <= B200_ACT_RELU, "hybrid_set_layer: unknown activation %d", w->act);
        m->layers[layer] = *w;
        if (w->side) {
            m->sides[layer] = *w->side;
            m->layers[layer].side = &m->sides[layer];
        }
        m->layer_set[layer] = 1;
        for (LayerPlan &lp : m->plan)
            if (lp.layer == layer) lp.n_in = n_in_of(m->layers[layer]);
        m->scratch = nullptr;
        return B200_OK;
    }
    B200_REQUIRE(w->mixer <= B200_MIXER_LATENT && !w->side, "hybrid_set_layer: mixer kind %d needs the shared-norm or the pre-norm layer form", w->mixer);
    B200_REQUIRE(m->cfg.loop_times == 0, "hybrid_set_layer: only shared-norm and pre-norm layers can be looped");
    if (w->norm == B200_NORM_RMS_POST) B200_REQUIRE(w->norm1, "hybrid_set_layer: norm weight missing");
    else B200_REQUIRE(w->pre1 && w->post1, "hybrid_set_layer: norm parameters missing");
    if (w->mixer == B200_MIXER_ATTN_CHUNKED) {
        B200_REQUIRE(w->kv_heads > 0 && w->heads % w->kv_heads == 0, "hybrid_set_layer: heads %d not a multiple of kv_heads %d", w->heads, w->kv_heads);
        B200_REQUIRE(w->vdim == w->dim, "hybrid_set_layer: this attention's values are its keys: vdim %d must equal dim %d", w->vdim, w->dim);
        B200_REQUIRE(w->chunk >= 0, "hybrid_set_layer: negative chunk");
    } else if (w->mixer == B200_MIXER_LATENT) {
        B200_REQUIRE(w->vdim > 0 && w->kv_rank > 0 && w->rot_dim >= 0 && w->window >= 0, "hybrid_set_layer: latent attention sizes missing");
        B200_REQUIRE(w->rot_dims >= 0 && w->rot_dims <= w->rot_dim && w->rot_dims % 2 == 0 && (w->rot_dims == 0 || w->rot_base > 0.0f),
                     "hybrid_set_layer: %d rotating dimensions do not fit a rotated part of %d (even, with a positive base)", w->rot_dims, w->rot_dim);
        B200_REQUIRE(w->w_uk_t && w->w_uv, "hybrid_set_layer: latent attention up-projections missing");
        B200_REQUIRE(w->kv_from < layer, "hybrid_set_layer: layer %d cannot read the latent rows of layer %d", layer, w->kv_from);
        B200_REQUIRE(w->kv_from >= 0 || w->kv_norm, "hybrid_set_layer: latent row norm weight missing");
    } else {
        B200_REQUIRE(w->vdim > 0 && w->decay_rank > 0 && w->tau > 0.0f && w->w_decay && w->out_norm, "hybrid_set_layer: gla sizes / weights missing");
    }
    B200_REQUIRE(w->mlp == B200_MLP_NONE || w->mlp == B200_MLP_MOE || w->mlp == B200_MLP_DENSE, "hybrid_set_layer: unknown feed-forward kind %d", w->mlp);
    if (w->mlp != B200_MLP_NONE) {
        if (w->norm == B200_NORM_RMS_POST) B200_REQUIRE(w->norm2, "hybrid_set_layer: feed-forward norm weight missing");
        else B200_REQUIRE(w->pre2 && w->post2, "hybrid_set_layer: feed-forward norm parameters missing");
        B200_REQUIRE(w->act >= B200_ACT_RELU2 && w->act <= B200_ACT_RELU, "hybrid_set_layer: unknown activation %d", w->act);
        B200_REQUIRE(w->expert_ff > 0 && w->w_up && w->w_down, "hybrid_set_layer: feed-forward sizes / weights missing");
    }
    if (w->mlp == B200_MLP_MOE) {
        B200_REQUIRE(w->experts > 0 && w->top > 0 && w->shared_ff >= 0 && w->identity >= 0, "hybrid_set_layer: bad expert counts");
        B200_REQUIRE(w->route == B200_ROUTE_SIGMOID || w->route == B200_ROUTE_SOFTMAX, "hybrid_set_layer: unknown router kind %d", w->route);
        if (w->route == B200_ROUTE_SIGMOID) {
            B200_REQUIRE(w->top <= w->experts && w->identity == 0 && !w->gated, "hybrid_set_layer: the sigmoid router has no identity or gated experts");
            B200_REQUIRE(w->norm == B200_NORM_RMS_POST, "hybrid_set_layer: the sigmoid router weighs the fp32 residual row: post-norm layers only");
        } else {
            B200_REQUIRE(w->top <= w->experts + w->identity, "hybrid_set_layer: top %d of %d router outputs", w->top, w->experts + w->identity);
        }
        B200_REQUIRE(w->w_router, "hybrid_set_layer: router weights missing");
        B200_REQUIRE(w->shared_ff == 0 || (w->w_shared_up && w->w_shared_down), "hybrid_set_layer: shared expert weights missing");
    }
    m->layers[layer] = *w;
    m->layer_set[layer] = 1;
    m->plan[layer].n_in = n_in_of(*w);  // (no loop here: run == layer)
    m->scratch = nullptr;  // sizes may have changed
    return B200_OK;
}

int b200_hybrid_set_io(b200_hybrid_t *m, const void *embedding, const float *final_norm, const void *lm_head) {
    B200_REQUIRE(m && embedding && final_norm && lm_head, "hybrid_set_io: null argument");
    m->embedding = embedding, m->final_norm = final_norm, m->lm_head = lm_head;
    return B200_OK;
}

int b200_hybrid_set_loop(b200_hybrid_t *m, const void *w_entry, const float *step) {
    B200_REQUIRE(m && w_entry && step, "hybrid_set_loop: null argument");
    B200_REQUIRE(m->cfg.loop_times > 0, "hybrid_set_loop: the engine was created without a looped block");
    m->w_entry = w_entry, m->loop_step = step;
    return B200_OK;
}

int b200_hybrid_num_runs(const b200_hybrid_t *m) { return m ? (int)m->plan.size() : 0; }

size_t b200_hybrid_scratch_bytes(const b200_hybrid_t *m) { return m ? carve(m).total : 0; }

int b200_hybrid_set_scratch(b200_hybrid_t *m, void *ptr, size_t bytes) {
    B200_REQUIRE(m && ptr, "hybrid_set_scratch: null argument");
    B200_REQUIRE(((uintptr_t)ptr & 255) == 0, "hybrid_set_scratch: pointer must be 256-byte aligned");
    for (int i = 0; i < m->cfg.num_layers; ++i) B200_REQUIRE(m->layer_set[i], "hybrid_set_scratch: layer %d not set", i);
    const Carve k = carve(m);
    B200_REQUIRE(bytes >= k.total, "hybrid_set_scratch: need %zu bytes, got %zu", k.total, bytes);
    char *p = (char *)ptr;
    m->scratch = p;
    m->x = (float *)p, p += k.x;
    m->f32a = (float *)p, p += k.f32a;
    m->f32b = (float *)p, p += k.f32b;
    m->xn = (float *)p, p += k.xn;
    m->h = p, p += k.h;
    m->proj = p, p += k.proj;
    m->mix = p, p += k.mix;
    m->mix2 = p, p += k.mix;
    m->y = p, p += k.y;
    m->xg = p, p += k.xg;
    m->u = p, p += k.u;
    m->yrows = p, p += k.yrows;
    m->us = p, p += k.us;
    m->ys = p, p += k.ys;
    m->lqn = p, p += k.lqn;
    m->lqr = p, p += k.lqr;
    m->lql = p, p += k.lql;
    m->lol = p, p += k.lql;
    m->lov = p, p += k.lov;
    m->lpart = (float *)p, p += k.lpart;
    m->meta = (int *)p, p += k.meta;
    m->moe_i = (int *)p, p += k.moe_i;
    m->moe_f = (float *)p, p += k.moe_f;
    m->rec = (float *)p, p += k.rec;
    m->f32c = (float *)p, p += k.f32c;
    m->cat = p, p += k.cat;
    m->xc = p, p += k.xc;
    m->xs = (float *)p, p += k.xs;
    return B200_OK;
}

namespace {
// what one mixer of one run takes from the two pools; `plan` (optional) receives the offsets
void place_mixer(const b200_hybrid_layer_t &l, size_t es, int num_pages, int num_slots, size_t &kv, size_t &stt, MixerPlan *plan) {
    MixerPlan p;
    if (l.mixer == B200_MIXER_ATTN_CHUNKED) {
        const size_t one = align256((size_t)num_pages * l.kv_heads * kPageH * l.dim * es);
        p.k_off = kv, p.v_off = kv + one, kv += 2 * one;
    } else if (l.mixer == B200_MIXER_ATTN_SCORED) {
        p.k_off = kv, kv += align256((size_t)num_pages * l.kv_heads * kPageH * l.dim * es);
        p.v_off = kv, kv += align256((size_t)num_pages * l.kv_heads * kPageH * l.vdim * es);
    } else if (l.mixer == B200_MIXER_LATENT) {
        if (l.kv_from < 0) p.k_off = kv, kv += align256((size_t)num_pages * kPageH * (l.kv_rank + l.rot_dim) * es);
    } else {
        p.state_off = stt, stt += align256((size_t)num_slots * l.heads * l.dim * l.vdim * 4);
        if (l.mixer == B200_MIXER_DELTA || l.mixer == B200_MIXER_SSD) {
            p.aux_off = stt, stt += align256((size_t)num_slots * std::max(l.conv - 1, 1) * conv_channels(l) * 4);
        } else if (l.mixer == B200_MIXER_MLSTM) {
            p.aux_off = stt, stt += align256((size_t)num_slots * l.heads * l.dim * 4);
            p.aux2_off = stt, stt += align256((size_t)num_slots * l.heads * 4);
        }
    }
    if (plan) *plan = p;
}
}  // namespace

size_t b200_hybrid_kv_pool_bytes(const b200_hybrid_t *m, int num_pages) {
    if (!m || num_pages <= 0) return 0;
    const size_t es = m->cfg.dtype == B200_F32 ? 4 : 2;
    size_t kv = 0, stt = 0;
    for (const LayerPlan &lp : m->plan) {
        if (!m->layer_set[lp.layer]) continue;
        place_mixer(m->layers[lp.layer], es, num_pages, 1, kv, stt, nullptr);
        if (m->layers[lp.layer].side) place_mixer(*m->layers[lp.layer].side, es, num_pages, 1, kv, stt, nullptr);
    }
    return kv ? kv : 256;
}

size_t b200_hybrid_state_pool_bytes(const b200_hybrid_t *m, int num_slots) {
    if (!m || num_slots <= 0) return 0;
    size_t kv = 0, stt = 0;
    for (const LayerPlan &lp : m->plan) {
        if (!m->layer_set[lp.layer]) continue;
        place_mixer(m->layers[lp.layer], 2, 1, num_slots, kv, stt, nullptr);
        if (m->layers[lp.layer].side) place_mixer(*m->layers[lp.layer].side, 2, 1, num_slots, kv, stt, nullptr);
    }
    return stt ? stt : 256;
}

int b200_hybrid_set_pools(b200_hybrid_t *m, void *kv_pool, int num_pages, void *state_pool, int num_slots) {
    B200_REQUIRE(m && kv_pool && state_pool && num_pages > 0 && num_slots > 0, "hybrid_set_pools: bad argument");
    B200_REQUIRE(((uintptr_t)kv_pool & 255) == 0 && ((uintptr_t)state_pool & 255) == 0, "hybrid_set_pools: pools must be 256-byte aligned");
    const size_t es = m->cfg.dtype == B200_F32 ? 4 : 2;
    size_t kv = 0, stt = 0;
    for (size_t r = 0; r < m->plan.size(); ++r) {
        LayerPlan &lp = m->plan[r];
        const int i = lp.layer;
        B200_REQUIRE(m->layer_set[i], "hybrid_set_pools: layer %d not set", i);
        const b200_hybrid_layer_t &l = m->layers[i];
        place_mixer(l, es, num_pages, num_slots, kv, stt, &lp);
        if (l.side) place_mixer(*l.side, es, num_pages, num_slots, kv, stt, &lp.side);
        if (l.mixer == B200_MIXER_LATENT && l.kv_from >= 0) {  // the rows of an earlier layer, which must own them and rotate them alike
            const b200_hybrid_layer_t &o = m->layers[l.kv_from];
            B200_REQUIRE(o.mixer == B200_MIXER_LATENT && o.kv_from < 0 && o.kv_rank == l.kv_rank && o.rot_dim == l.rot_dim &&
                             o.rot_dims == l.rot_dims && o.rot_base == l.rot_base,
                         "hybrid_set_pools: layer %d cannot read the latent rows of layer %d (no cache of its own, or other sizes)", i, l.kv_from);
            lp.k_off = m->plan[l.kv_from].k_off;  // (latent layers are never looped: run == layer)
        }
    }
    m->kv_pool = (char *)kv_pool, m->state_pool = (char *)state_pool, m->num_pages = num_pages, m->num_slots = num_slots;
    return B200_OK;
}

int b200_hybrid_forward(b200_hybrid_t *m, const b200_hybrid_batch_t *b, float *logits, float *layer_trace, b200_stream_t stream) {
    B200_REQUIRE(m && b, "hybrid_forward: null argument");
    if (!m->scratch || !m->kv_pool || !m->embedding) {
        set_error("hybrid_forward: scratch, pools or embedding / head not set");
        return B200_ERR_STATE;
    }
    const b200_hybrid_config_t &c = m->cfg;
    const int NT = b->n_tokens, S = b->n_seqs, W = b->n_want, mpps = c.max_pages_per_seq;
    B200_REQUIRE(NT >= 0 && NT <= c.max_tokens && S >= 0 && S <= c.max_seqs && W >= 0 && W <= NT, "hybrid_forward: %d tokens / %d sequences / %d wanted rows outside the engine's limits (%d, %d)",
                 NT, S, W, c.max_tokens, c.max_seqs);
    if (NT == 0) return B200_OK;
    B200_REQUIRE(b->token_ids && b->seq_start && b->seq_pos0 && b->seq_slot && b->block_table && (W == 0 || (b->want_rows && logits)),
                 "hybrid_forward: null batch array");
    B200_REQUIRE(b->seq_start[0] == 0 && b->seq_start[S] == NT, "hybrid_forward: seq_start must run from 0 to n_tokens");

    // ---- batch description: checked on the host, shipped in one copy
    std::vector<int> &hm = m->host_meta;
    // latent mixers: their per-head products are grouped GEMMs over [heads, t_pad, *]; row tile i belongs to head i / (tiles per head).
    // Prompt-sized batches of a 16-bit engine take 128-row tiles on the tcgen05 grouped GEMM, others 64-row tiles on mma.sync / SIMT.
    int lat_heads = 0;
    bool lat_by_head = false;  // some latent layer runs its short portions as one-token tiles over 64 heads
    for (int i = 0; i < c.num_layers; ++i) {
        const b200_hybrid_layer_t &l = m->layers[i];
        if (l.mixer != B200_MIXER_LATENT) continue;
        lat_heads = std::max(lat_heads, l.heads);
        lat_by_head |= l.heads >= kLatentHeadsPerTile && latent_attention_tiles_supported(c.dtype, l.kv_rank, l.rot_dim);
    }
    const bool lat_tc = c.dtype != B200_F32 && NT >= 256;
    const int t_pad = lat_tc ? (NT + 127) / 128 * 128 : (NT + kMoeTileM - 1) / kMoeTileM * kMoeTileM;
    const int tph = t_pad / kMoeTileM, tph128 = lat_tc ? t_pad / 128 : 0;
    const size_t n_tile_ints = 4 * ((size_t)NT / 64 + S + 1), n_stile_ints = lat_by_head ? (size_t)4 * NT : 0;
    hm.assign(n_tile_ints + n_stile_ints + (size_t)5 * NT + 3 * S + 1 + (size_t)S * mpps + (size_t)lat_heads * (tph + tph128) + 2 * c.num_layers, 0);
    int *h_tiles = hm.data(), *h_stiles = h_tiles + n_tile_ints, *h_ids = h_stiles + n_stile_ints, *h_seq = h_ids + NT, *h_pos = h_seq + NT,
        *h_want = h_pos + NT, *h_short = h_want + NT, *h_start = h_short + NT, *h_pos0 = h_start + S + 1, *h_slot = h_pos0 + S, *h_bt = h_slot + S,
        *h_lat_head = h_bt + (size_t)S * mpps, *h_lat_head128 = h_lat_head + (size_t)lat_heads * tph,
        *h_lat_n = h_lat_head128 + (size_t)lat_heads * tph128, *h_lat_n128 = h_lat_n + c.num_layers;
    for (int i = 0; i < lat_heads * tph; ++i) h_lat_head[i] = i / tph;
    for (int i = 0; i < lat_heads * tph128; ++i) h_lat_head128[i] = i / tph128;
    for (int i = 0; i < c.num_layers; ++i) {
        const bool lat = m->layers[i].mixer == B200_MIXER_LATENT;
        h_lat_n[i] = lat ? m->layers[i].heads * tph : 0, h_lat_n128[i] = lat ? m->layers[i].heads * tph128 : 0;
    }
    // prompt portions go to the tensor-core attention in tiles of <= 64 consecutive tokens, short ones (decoded tokens) to the per-token kernel
    constexpr int kShortPortion = 8;
    int n_tiles = 0, n_short = 0, gla_kinds = 0;
    for (int s = 0; s < S; ++s) {
        const int t0 = b->seq_start[s], t1 = b->seq_start[s + 1];
        gla_kinds |= t1 - t0 == 1 ? kGlaOneToken : (t1 - t0 > 1 ? kGlaManyTokens : 0);
        B200_REQUIRE(t1 >= t0 && b->seq_pos0[s] >= 0, "hybrid_forward: bad portion of sequence %d", s);
        B200_REQUIRE(b->seq_slot[s] >= 0 && b->seq_slot[s] < m->num_slots, "hybrid_forward: state slot %d outside [0, %d)", b->seq_slot[s], m->num_slots);
        for (int s2 = 0; s2 < s; ++s2) B200_REQUIRE(b->seq_slot[s2] != b->seq_slot[s], "hybrid_forward: state slot %d given to two sequences", b->seq_slot[s]);
        const int last = b->seq_pos0[s] + (t1 - t0) - 1;
        B200_REQUIRE(last < mpps * kPageH, "hybrid_forward: position %d exceeds a block-table row (%d pages)", last, mpps);
        for (int p = 0; p <= last / kPageH && t1 > t0; ++p) {
            const int page = b->block_table[(size_t)s * mpps + p];
            B200_REQUIRE(page >= 0 && page < m->num_pages, "hybrid_forward: sequence %d holds no page for positions %d..", s, p * kPageH);
        }
        for (int t = t0; t < t1; ++t) h_seq[t] = s, h_pos[t] = b->seq_pos0[s] + (t - t0);
        if (t1 - t0 < kShortPortion) {
            for (int t = t0; t < t1; ++t) {
                if (lat_by_head) {
                    int *tl = h_stiles + 4 * n_short;
                    tl[0] = s, tl[1] = t, tl[2] = 1, tl[3] = h_pos[t];
                }
                h_short[n_short++] = t;
            }
        } else {
            for (int t = t0; t < t1; t += 64, ++n_tiles) {
                int *tl = h_tiles + 4 * n_tiles;
                tl[0] = s, tl[1] = t, tl[2] = std::min(64, t1 - t), tl[3] = h_pos[t];
            }
        }
        h_start[s] = t0, h_pos0[s] = b->seq_pos0[s], h_slot[s] = b->seq_slot[s];
        for (int p = 0; p < mpps; ++p) h_bt[(size_t)s * mpps + p] = b->block_table[(size_t)s * mpps + p];
    }
    h_start[S] = NT;
    for (int t = 0; t < NT; ++t) {
        B200_REQUIRE(b->token_ids[t] >= 0 && b->token_ids[t] < c.vocab, "hybrid_forward: token id %d outside the vocabulary", b->token_ids[t]);
        h_ids[t] = b->token_ids[t];
    }
    for (int i = 0; i < W; ++i) {
        B200_REQUIRE(b->want_rows[i] >= 0 && b->want_rows[i] < NT, "hybrid_forward: wanted row %d outside the batch", b->want_rows[i]);
        h_want[i] = b->want_rows[i];
    }
    cudaStream_t st = as_stream(stream);
    NvtxRange range("hybrid_forward");
    if (cudaMemcpyAsync(m->meta, hm.data(), hm.size() * sizeof(int), cudaMemcpyHostToDevice, st) != cudaSuccess) return cuda_status("hybrid_forward meta copy");
    const int *d_tiles = m->meta, *d_stiles = d_tiles + n_tile_ints, *d_ids = d_stiles + n_stile_ints, *d_seq = d_ids + NT, *d_pos = d_seq + NT,
              *d_want = d_pos + NT, *d_short = d_want + NT, *d_start = d_short + NT, *d_pos0 = d_start + S + 1, *d_slot = d_pos0 + S, *d_bt = d_slot + S,
              *d_lat_head = d_bt + (size_t)S * mpps, *d_lat_head128 = d_lat_head + (size_t)lat_heads * tph,
              *d_lat_n = d_lat_head128 + (size_t)lat_heads * tph128, *d_lat_n128 = d_lat_n + c.num_layers;

    const int dt = c.dtype, width = c.width;
    const bool f32 = dt == B200_F32;
    int rc;
#define RUN(expr)                    \
    do {                             \
        rc = (expr);                 \
        if (rc != B200_OK) return rc; \
    } while (0)
    // 16-bit engines: every kernel that writes the residual stream also writes its 16-bit copy h, which the next projections read
    const int n_runs = (int)m->plan.size();
    const bool shared_norm = m->layers[0].norm == B200_NORM_LN_PARALLEL;  // layers of one norm whose sublayers share the projections
    const bool pre_norm = m->layers[0].norm == B200_NORM_LN_PRE;          // pre-norm layers on residual streams
    for (int i = 0; i < c.num_layers; ++i)
        B200_REQUIRE((m->layers[i].norm == B200_NORM_LN_PARALLEL) == shared_norm && (m->layers[i].norm == B200_NORM_LN_PRE) == pre_norm,
                     "hybrid_forward: shared-norm layers, pre-norm layers and others do not mix in one model");
    if (shared_norm && c.loop_times > 0 && (!m->w_entry || !m->loop_step)) {
        set_error("hybrid_forward: the looped block's entry weights are not set");
        return B200_ERR_STATE;
    }
    const size_t es = f32 ? 4 : 2;
    // the residual step of a shared-norm layer; it also writes what the next run reads: its normed input, or (before an entry step) x itself
    auto ln_residual = [&](const void *y, const float *y32, const float *bias, const float *ln, void *h_out, int h_ld, float *trace) -> int {
        B200_DISPATCH_DTYPE(dt, {
            ln_residual_kernel<T><<<NT, 256, (size_t)width * sizeof(float), st>>>(m->x, (const T *)y, y32, bias, y32 ? 1 : 0, ln, c.norm_eps, width,
                                                                                (T *)h_out, h_ld, trace);
        });
        return cuda_status("ln_residual launch");
    };
    // hands x over to run `run`: the normed input of its layer, or x itself into the left half of the entry step's input row
    auto hand_over = [&](int run, const void *y, const float *bias, float *trace) -> int {
        if (run >= n_runs) return (y || bias || trace) ? ln_residual(y, nullptr, bias, nullptr, nullptr, 0, trace) : B200_OK;
        if (m->plan[run].entry >= 0) return ln_residual(y, nullptr, bias, nullptr, m->xc, 2 * width, trace);
        return ln_residual(y, nullptr, bias, m->layers[m->plan[run].layer].pre1, m->h, width, trace);
    };
    if (shared_norm) {
        B200_DISPATCH_DTYPE(dt, {
            embed_rows_kernel<T><<<NT, 128, 0, st>>>(d_ids, (const T *)m->embedding, m->x, c.loop_times > 0 ? (T *)m->xc + width : nullptr, 2 * width, width,
                                                    c.vocab, c.embed_scale != 0.0f ? c.embed_scale : 1.0f);
        });
        RUN(hand_over(0, nullptr, nullptr, nullptr));
    } else if (pre_norm) {
        B200_DISPATCH_DTYPE(dt, {
            embed_rows_kernel<T><<<NT, 128, 0, st>>>(d_ids, (const T *)m->embedding, m->x, (T *)nullptr, 0, width, c.vocab, c.embed_scale != 0.0f ? c.embed_scale : 1.0f);
        });
    } else {
    B200_DISPATCH_DTYPE(dt, { embed_f32_kernel<T><<<NT, 128, 0, st>>>(d_ids, (const T *)m->embedding, m->x, f32 ? nullptr : (T *)m->h, width, c.vocab,
                                                                      c.embed_scale != 0.0f ? c.embed_scale : 1.0f); });
    }

    // one mixer of a shared-norm or pre-norm layer: reads its rows of the projection from column `col`, writes its heads into rows of `out`
    // (row stride out_ld: several mixers may fill one row of a shared output projection's input), scaled
    auto run_mixer = [&](const b200_hybrid_layer_t &l, const MixerPlan &mp, int n_in, int col, void *out_buf, int out_ld, float out_scale) -> int {
        char *out = (char *)out_buf;
        const int one_token = gla_kinds == kGlaOneToken;
        if (l.mixer == B200_MIXER_ATTN_SCORED) {
            const char *gate = l.out_gate ? (const char *)m->proj + (size_t)(col + (l.heads + l.kv_heads) * l.dim + l.kv_heads * l.vdim) * es : nullptr;
            char *kp = m->kv_pool + mp.k_off, *vp = m->kv_pool + mp.v_off;
            const int sig = l.attn_weight == B200_ATTN_SIGMOID;
            ScoredPrepOptions opt;
            opt.rot_half = l.rot_half, opt.rot_factor = l.rot_factor, opt.rot_low = l.rot_low, opt.rot_high = l.rot_high, opt.rot_original = l.rot_original;
            opt.v_norm = l.v_norm;
            RUN(launch_scored_prep(dt, m->proj, n_in, col, l.b_in, m->mix, kp, vp, l.q_norm, l.k_norm, c.norm_eps, d_seq, d_pos, d_bt, mpps, NT, l.heads,
                                   l.kv_heads, l.dim, l.vdim, l.rot_dims, l.rot_base, st, opt));
            const int max_keys = l.window > 0 ? std::min(l.window, mpps * kPageH) : mpps * kPageH;
            if (scored_attention_tiles_supported(dt, l.dim, l.vdim, n_in, out_ld, l.window, l.dist_r1 != nullptr)) {
                RUN(launch_scored_attention_tiles(dt, m->mix, kp, vp, l.head_bias, l.dist_r1, l.dist_r2, gate, n_in, out, out_ld, out_scale, d_tiles, n_tiles,
                                                  d_bt, mpps, l.heads, l.kv_heads, l.dim, l.vdim, l.scale, l.window, sig, st, l.softcap));
                RUN(launch_scored_attention(dt, m->mix, kp, vp, l.head_bias, l.dist_r1, l.dist_r2, gate, n_in, out, out_ld, out_scale, d_seq, d_pos, d_bt,
                                            mpps, n_short, l.heads, l.kv_heads, l.dim, l.vdim, l.scale, l.window, sig, max_keys, st, d_short, l.softcap));
            } else {
                RUN(launch_scored_attention(dt, m->mix, kp, vp, l.head_bias, l.dist_r1, l.dist_r2, gate, n_in, out, out_ld, out_scale, d_seq, d_pos, d_bt,
                                            mpps, NT, l.heads, l.kv_heads, l.dim, l.vdim, l.scale, l.window, sig, max_keys, st, nullptr, l.softcap));
            }
        } else if (l.mixer == B200_MIXER_DELTA) {
            float *conv_state = (float *)(m->state_pool + mp.aux_off);
            const DeltaRow lay = delta_row(l.heads, l.kv_heads, l.dim, l.vdim);
            if (l.decay_rank > 0)
                RUN(launch_delta_prep(dt, m->proj, n_in, col, l.conv_w, l.conv, conv_state, l.w_decay, l.decay_bias, l.a_log, l.decay_rank, l.w_gate2,
                                      l.gate_rank, m->mix2, m->f32a, m->f32b, m->rec, d_seq, d_pos, d_pos0, d_slot, NT, l.heads, l.kv_heads, l.dim, l.vdim, st));
            else
                RUN(launch_delta_prep_direct(dt, m->proj, n_in, col, l.conv_w, l.conv, conv_state, l.decay_bias, l.a_log, m->rec, d_seq, d_pos, d_pos0, d_slot,
                                             NT, l.heads, l.kv_heads, l.dim, l.vdim, st));
            RUN(launch_conv_state_update(dt, m->proj, n_in, col, conv_state, l.conv, conv_channels(l), d_start, d_pos0, d_slot, S, st));
            RUN(launch_delta_recurrent(m->rec, (float *)(m->state_pool + mp.state_off), m->f32b, d_start, d_pos0, d_slot, S, l.heads, l.kv_heads, l.dim,
                                       l.vdim, st, one_token));
            if (l.decay_rank > 0) {
                RUN(launch_head_output(dt, m->f32b, nullptr, nullptr, l.out_norm, 0, c.norm_eps, m->rec + lay.gate, lay.ld, nullptr, 0, out, out_ld, out_scale,
                                       NT, l.heads, l.vdim, st, l.gate_act));
            } else {  // the gate's pre-activations are rows of the projection
                const char *gate = (const char *)m->proj + (size_t)(col + conv_channels(l) + 2 * l.heads) * es;
                RUN(launch_head_output(dt, m->f32b, nullptr, nullptr, l.out_norm, 0, c.norm_eps, nullptr, 0, gate, n_in, out, out_ld, out_scale, NT, l.heads,
                                       l.vdim, st, l.gate_act));
            }
        } else if (l.mixer == B200_MIXER_SSD) {
            // z | x | B | C | dt: the convolution runs over x | B | C; the recurrence's key side is B (per group), its query side C
            float *conv_state = (float *)(m->state_pool + mp.aux_off);
            const int inner = l.heads * l.vdim;
            const DecayRow lay = decay_row(l.heads, l.kv_heads, l.dim, l.vdim);
            RUN(launch_ssd_prep(dt, m->proj, n_in, col, l.conv_w, l.conv_b, l.conv, conv_state, l.decay_bias, l.a_log, l.skip, m->rec, d_seq, d_pos, d_pos0,
                                d_slot, NT, l.heads, l.kv_heads, l.dim, l.vdim, st));
            RUN(launch_conv_state_update(dt, m->proj, n_in, col + inner, conv_state, l.conv, conv_channels(l), d_start, d_pos0, d_slot, S, st));
            RUN(launch_decay_recurrent(m->rec, (float *)(m->state_pool + mp.state_off), m->f32b, d_start, d_pos0, d_slot, S, l.heads, l.kv_heads, l.dim,
                                       l.vdim, st, one_token));
            RUN(launch_group_output(dt, m->f32b, m->rec + lay.skip, lay.ld, l.out_norm, c.norm_eps, (const char *)m->proj + (size_t)col * es, n_in, 1, 1, out,
                                    out_ld, NT, inner, l.norm_groups, st));
        } else if (l.mixer == B200_MIXER_LINEAR) {
            const int inner = l.heads * l.vdim;
            RUN(launch_linear_prep(dt, m->proj, n_in, col, l.head_decay, m->rec, NT, l.heads, l.dim, l.vdim, st));
            RUN(launch_decay_recurrent(m->rec, (float *)(m->state_pool + mp.state_off), m->f32b, d_start, d_pos0, d_slot, S, l.heads, l.heads, l.dim, l.vdim,
                                       st, one_token));
            RUN(launch_group_output(dt, m->f32b, nullptr, 0, l.out_norm, c.norm_eps, (const char *)m->proj + (size_t)(col + 2 * l.heads * l.dim + inner) * es,
                                    n_in, 0, 0, out, out_ld, NT, inner, 1, st));
        } else {
            const char *gate = (const char *)m->proj + (size_t)(col + 2 * l.heads * l.dim + l.heads * l.vdim) * es;
            float *nq = m->f32c, *mo = m->f32c + (size_t)NT * l.heads;
            RUN(launch_mlstm_prep(dt, m->proj, n_in, col, l.b_in, l.gate_cap, m->rec, NT, l.heads, l.dim, l.vdim, st));
            RUN(launch_mlstm_recurrent(m->rec, (float *)(m->state_pool + mp.state_off), (float *)(m->state_pool + mp.aux_off),
                                       (float *)(m->state_pool + mp.aux2_off), m->f32b, nq, mo, d_start, d_pos0, d_slot, S, l.heads, l.dim, l.vdim, st, one_token));
            RUN(launch_head_output(dt, m->f32b, nq, mo, l.out_norm, l.vdim, c.norm_eps, nullptr, 0, gate, n_in, out, out_ld, out_scale, NT, l.heads, l.vdim, st));
        }
        return B200_OK;
    };
    // ---- pre-norm layers on residual streams
    const int n_streams = std::max(c.streams, 1);
    // the residual step of one sublayer + the layer-normed input of the sublayer that follows (hc_next / ln_next; none after the last run)
    auto stream_step = [&](const float *x_init, const void *ya, const void *yb, const float *na, const float *nb, float sa, float sb, const float *hc,
                           const float *hc_next, const float *ln_next, float *sum_out, float *trace) -> int {
        // four columns per access when every row starts on a 16-byte boundary (the scratch buffers do; norm vectors and the trace are the caller's)
        const bool vec = width % 4 == 0 && ((reinterpret_cast<size_t>(na) | reinterpret_cast<size_t>(nb) | reinterpret_cast<size_t>(ln_next) |
                                              reinterpret_cast<size_t>(trace)) & 15) == 0;
#define B200_STREAMS(SC, V) stream_residual_kernel<T, SC, V><<<NT, 256, (size_t)width * sizeof(float), st>>>(                                           \
    m->xs, n_streams, x_init, (const T *)ya, (const T *)yb, na, nb, sa, sb, hc, hc_next, ln_next, c.norm_eps, width, ln_next ? (T *)m->h : nullptr, sum_out, trace)
#define B200_STREAMS_V(SC) do { if (vec) B200_STREAMS(SC, true); else B200_STREAMS(SC, false); } while (0)
        B200_DISPATCH_DTYPE(dt, {
            switch (n_streams) {
                case 1: B200_STREAMS_V(1); break;
                case 2: B200_STREAMS_V(2); break;
                case 3: B200_STREAMS_V(3); break;
                case 4: B200_STREAMS_V(4); break;
                default: B200_STREAMS_V(0); break;
            }
        });
#undef B200_STREAMS_V
#undef B200_STREAMS
        return cuda_status("stream_residual launch");
    };
    auto pre_norm_layer = [&](int run) -> int {
        const LayerPlan &lp = m->plan[run];
        const b200_hybrid_layer_t &l = m->layers[lp.layer];
        const b200_hybrid_layer_t *next = run + 1 < n_runs ? &m->layers[m->plan[run + 1].layer] : nullptr;
        const bool last = next == nullptr, ff = l.mlp == B200_MLP_DENSE;
        float *trace = layer_trace ? layer_trace + (size_t)run * NT * width : nullptr;
        RUN(linear(m, m->h, l.w_in, m->proj, NT, width, lp.n_in, st));
        // every mixer has an output projection of its own: the first writes its heads to `cat`, the second to `mix2`
        RUN(run_mixer(l, lp, lp.n_in, 0, m->cat, l.heads * l.vdim, 1.0f));
        RUN(linear(m, m->cat, l.w_out, m->y, NT, l.heads * l.vdim, width, st));
        if (l.side) {
            RUN(run_mixer(*l.side, lp.side, lp.n_in, mixer_rows(l), m->mix2, l.side->heads * l.side->vdim, 1.0f));
            RUN(linear(m, m->mix2, l.side->w_out, m->ys, NT, l.side->heads * l.side->vdim, width, st));
        }
        RUN(stream_step(nullptr, m->y, l.side ? m->ys : nullptr, l.branch_norm, l.side ? l.side->branch_norm : nullptr, l.side ? l.mix_scale : 1.0f,
                        l.side ? l.side_scale : 1.0f, l.hc1, ff ? l.hc2 : (next ? next->hc1 : nullptr), ff ? l.pre2 : (next ? next->pre1 : nullptr),
                        (!ff && last) ? m->x : nullptr, ff ? nullptr : trace));
        if (!ff) return B200_OK;
        char *up = (char *)m->us, *act = up + (size_t)NT * 2 * l.expert_ff * es;
        RUN(linear(m, m->h, l.w_up, up, NT, width, 2 * l.expert_ff, st));
        RUN(launch_gated_activation(dt, up, act, NT, l.expert_ff, l.act, nullptr, 0, st));
        RUN(linear(m, act, l.w_down, m->ys, NT, l.expert_ff, width, st));
        return stream_step(nullptr, m->ys, nullptr, nullptr, nullptr, 1.0f, 1.0f, l.hc2, next ? next->hc1 : nullptr, next ? next->pre1 : nullptr,
                           last ? m->x : nullptr, trace);
    };
    if (pre_norm) RUN(stream_step(m->x, nullptr, nullptr, nullptr, nullptr, 1.0f, 1.0f, nullptr, m->layers[m->plan[0].layer].hc1, m->layers[m->plan[0].layer].pre1, nullptr, nullptr));
    // a shared-norm layer run: (entry step) -> one input projection -> mixers and the gated inner row side by side -> one output
    // projection -> residual + the next run's normed input
    auto shared_norm_layer = [&](int run) -> int {
        const LayerPlan &lp = m->plan[run];
        const b200_hybrid_layer_t &l = m->layers[lp.layer];
        if (lp.entry >= 0) {  // x <- w_entry [x ; x0] + step[pass], fp32 out; then this layer's norm
            // (a decode batch is a single row tile on the tensor-core kernel -- N / 128 CTAs, each walking all of K: it takes the row kernel)
            rc = NT > 16 ? launch_dense_f32out(dt, m->xc, m->w_entry, m->xn, NT, width, 2 * width, st) : B200_ERR_UNSUPPORTED;
            if (rc == B200_ERR_UNSUPPORTED) rc = launch_proj_f32(dt, m->xc, 2 * width, dt, m->w_entry, nullptr, m->xn, width, NT, width, 2 * width, st);
            if (rc != B200_OK) return rc;
            RUN(ln_residual(nullptr, m->xn, m->loop_step + (size_t)lp.entry * width, l.pre1, m->h, width, nullptr));
        }
        const int n_cat = cat_cols(l);
        RUN(linear(m, m->h, l.w_in, m->proj, NT, width, lp.n_in, st));
        int col = 0, ocol = 0;
        RUN(run_mixer(l, lp, lp.n_in, col, (char *)m->cat + (size_t)ocol * es, n_cat, l.side ? l.mix_scale : 1.0f));
        col += mixer_rows(l), ocol += l.heads * l.vdim;
        if (l.side) {
            RUN(run_mixer(*l.side, lp.side, lp.n_in, col, (char *)m->cat + (size_t)ocol * es, n_cat, l.side_scale));
            col += mixer_rows(*l.side), ocol += l.side->heads * l.side->vdim;
        }
        if (l.mlp == B200_MLP_DENSE) {
            B200_DISPATCH_DTYPE(dt, {
                constexpr int V = Elem<T>::kVec;
                const bool vec = lp.n_in % V == 0 && col % V == 0 && l.expert_ff % V == 0 && n_cat % V == 0 && ocol % V == 0;
                const int per = vec ? V : 1;
                const dim3 grid((l.expert_ff / per + 255) / 256, NT);
                if (vec) gated_act_strided_kernel<T, true><<<grid, 256, 0, st>>>((const T *)m->proj, lp.n_in, col, col + l.expert_ff, (T *)m->cat + ocol, n_cat, l.expert_ff, l.act);
                else gated_act_strided_kernel<T, false><<<grid, 256, 0, st>>>((const T *)m->proj, lp.n_in, col, col + l.expert_ff, (T *)m->cat + ocol, n_cat, l.expert_ff, l.act);
            });
            RUN(cuda_status("gated_act_strided launch"));
        }
        RUN(linear(m, m->cat, l.w_out, m->y, NT, n_cat, width, st));
        return hand_over(run + 1, m->y, l.b_out, layer_trace ? layer_trace + (size_t)run * NT * width : nullptr);
    };

    auto cast_x = [&]() -> const void * { return f32 ? (const void *)m->x : (const void *)m->h; };
    auto postnorm = [&](const void *y_dense, const void *y_rows, const int *pair_row, int top, const void *y_shared, const float *gate,
                        const float *g, float *trace) -> int {
        B200_DISPATCH_DTYPE(dt, {
            postnorm_residual_kernel<T><<<NT, 256, (size_t)width * sizeof(float), st>>>(m->x, (const T *)y_dense, (const T *)y_rows, pair_row, top,
                                                                                      (const T *)y_shared, gate, g, c.norm_eps, width, trace,
                                                                                      f32 ? nullptr : (T *)m->h);
        });
        return cuda_status("postnorm_residual launch");
    };

    // the general residual kernel: either norm kind, routing weights on the outputs, identity experts, the next sublayer's pre-norm fused
    auto residual = [&](bool has_y, const void *y_dense, const float *y_bias, const void *y_rows, const int *pair_row, const float *pair_weight, int top,
                        const void *y_shared, const float *gate, int norm, const float *post, const float *ls, const float *pre, float *trace) -> int {
        B200_DISPATCH_DTYPE(dt, {
            // 16-byte pieces when every row starts on a 16-byte boundary (the scratch buffers do; the trace is the caller's)
            const bool vec = width % Elem<T>::kVec == 0 && ((reinterpret_cast<size_t>(trace) | reinterpret_cast<size_t>(post) | reinterpret_cast<size_t>(ls) |
                                                              reinterpret_cast<size_t>(pre) | reinterpret_cast<size_t>(y_bias)) & 15) == 0;
            auto kern = vec ? sublayer_residual_kernel<T, true> : sublayer_residual_kernel<T, false>;
            kern<<<NT, 256, (size_t)width * sizeof(float), st>>>(m->x, (const T *)y_dense, y_bias, (const T *)y_rows, pair_row, pair_weight, top,
                                                                (const T *)y_shared, gate, (const T *)m->h, norm, post, ls, c.norm_eps, pre, width, trace,
                                                                (pre || !f32) ? (T *)m->h : nullptr, has_y ? 1 : 0);
        });
        return cuda_status("sublayer_residual launch");
    };
    // the pre-norm of the sublayer that follows sublayer `sub` (0: mixer, 1: feed-forward) of layer li, or NULL
    auto next_pre = [&](int li, int sub) -> const float * {
        const b200_hybrid_layer_t &l = m->layers[li];
        if (sub == 0 && l.mlp != B200_MLP_NONE) return l.norm == B200_NORM_DYT_PRE_POST ? l.pre2 : nullptr;
        if (li + 1 >= c.num_layers) return nullptr;
        return m->layers[li + 1].norm == B200_NORM_DYT_PRE_POST ? m->layers[li + 1].pre1 : nullptr;
    };
    bool h_normed = false;  // m->h holds the pre-normed input of the coming sublayer

    for (int li = 0; li < n_runs; ++li) {  // (only shared-norm layers loop: elsewhere a run is its layer)
        if (shared_norm) {
            RUN(shared_norm_layer(li));
            continue;
        }
        if (pre_norm) {
            RUN(pre_norm_layer(li));
            continue;
        }
        const b200_hybrid_layer_t &l = m->layers[li];
        const LayerPlan &lp = m->plan[li];
        const bool dyt = l.norm == B200_NORM_DYT_PRE_POST;
        float *trace = (layer_trace && l.mlp == B200_MLP_NONE) ? layer_trace + (size_t)li * NT * width : nullptr;
        if (dyt && !h_normed) RUN(residual(false, nullptr, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, l.norm, nullptr, nullptr, l.pre1, nullptr));
        const void *h = dyt ? (const void *)m->h : cast_x();
        RUN(linear(m, h, l.w_in, m->proj, NT, width, lp.n_in, st));
        int n_mixed = 0;  // columns of the mixer's result before the output projection
        if (l.mixer == B200_MIXER_ATTN_CHUNKED) {
            const int hd = l.heads * l.dim;
            const char *gate = (const char *)m->proj + (size_t)(l.heads + l.kv_heads) * l.dim * es;
            RUN(launch_attn_qk_norm_cache(dt, m->proj, lp.n_in, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.q_norm, l.k_norm, c.norm_eps,
                                          d_seq, d_pos, d_bt, mpps, NT, l.heads, l.kv_heads, l.dim, st));
            const int max_keys = l.chunk > 0 ? l.chunk : mpps * kPageH;
            if (chunked_attention_tiles_supported(dt, l.dim, lp.n_in)) {
                RUN(launch_chunked_attention_tiles(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_tiles,
                                                   n_tiles, d_bt, mpps, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, st));
                RUN(launch_chunked_attention(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_seq, d_pos,
                                             d_bt, mpps, n_short, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, max_keys, st, d_short));
            } else {
                RUN(launch_chunked_attention(dt, m->mix, m->kv_pool + lp.k_off, m->kv_pool + lp.v_off, l.sink, gate, lp.n_in, m->mix2, d_seq, d_pos,
                                             d_bt, mpps, NT, l.heads, l.kv_heads, l.dim, l.scale, l.chunk, max_keys, st));
            }
            n_mixed = hd;
        } else if (l.mixer == B200_MIXER_LATENT) {
            const int nq = l.heads * (l.dim + l.rot_dim), hv = l.heads * l.vdim;
            const char *gate = (const char *)m->proj + (size_t)nq * es;
            char *pool = m->kv_pool + lp.k_off;
            RUN(launch_latent_prep(dt, m->proj, lp.n_in, 0, l.kv_from < 0 ? nq + hv : -1, m->lqn, m->lqr, pool, l.kv_norm, c.norm_eps, d_seq, d_pos, d_bt,
                                   mpps, NT, t_pad, l.heads, l.dim, l.rot_dim, l.kv_rank, l.rot_dims, l.rot_base, st));
            // the per-head products: rows past the batch's tokens hold whatever the scratch held; a row of a product depends on its own
            // input row only and those rows are never read
            auto head_product = [&](const void *a, const void *w, void *out, int N, int K) -> int {
                if (lat_tc) {
                    const int r = launch_gemm_tc_grouped(a, w, out, l.heads * t_pad, N, K, l.heads, d_lat_head128, d_lat_n128 + li, -1, dt, st);
                    if (r != B200_ERR_UNSUPPORTED) return r;
                }
                return launch_moe_grouped_gemm(dt, a, w, out, d_lat_head, d_lat_n + li, l.heads * tph, N, K, -1, st);
            };
            RUN(head_product(m->lqn, l.w_uk_t, m->lql, l.kv_rank, l.dim));  // q into the latent space: ql[h] = qn[h] . W_uk,h
            const int max_keys = l.window > 0 ? std::min(l.window, mpps * kPageH) : mpps * kPageH;
            if (latent_attention_tiles_supported(dt, l.kv_rank, l.rot_dim)) {
                RUN(launch_latent_attention_tiles(dt, m->lql, m->lqr, pool, l.sink, m->lol, d_tiles, n_tiles, d_bt, mpps, t_pad, l.heads, l.kv_rank,
                                                  l.rot_dim, l.scale, l.window, 0, nullptr, 0, st));
                // decoded tokens: one tile per token over its heads reads the window once per 64 heads (few tokens share out their keys over
                // several CTAs); layers of few heads take the per-token kernel, one CTA per (token, head)
                if (l.heads >= kLatentHeadsPerTile)
                    RUN(launch_latent_attention_tiles(dt, m->lql, m->lqr, pool, l.sink, m->lol, d_stiles, n_short, d_bt, mpps, t_pad, l.heads, l.kv_rank,
                                                      l.rot_dim, l.scale, l.window, 1, m->lpart, kLatentPartTiles, st));
                else
                    RUN(launch_latent_attention(dt, m->lql, m->lqr, pool, l.sink, m->lol, d_seq, d_pos, d_bt, mpps, n_short, t_pad, l.heads, l.kv_rank,
                                                l.rot_dim, l.scale, l.window, max_keys, st, d_short));
            } else {
                RUN(launch_latent_attention(dt, m->lql, m->lqr, pool, l.sink, m->lol, d_seq, d_pos, d_bt, mpps, NT, t_pad, l.heads, l.kv_rank, l.rot_dim,
                                            l.scale, l.window, max_keys, st));
            }
            RUN(head_product(m->lol, l.w_uv, m->lov, l.vdim, l.kv_rank));  // out[h] = (sum_j p c_j) . W_uv,h^T
            RUN(launch_latent_gate(dt, m->lov, gate, lp.n_in, m->mix2, NT, t_pad, l.heads, l.vdim, st));
            n_mixed = hv;
        } else {
            const int hd = l.heads * l.dim, hv = l.heads * l.vdim;
            const char *gate = (const char *)m->proj + (size_t)(2 * hd + hv) * es;
            RUN(launch_gla_decay(dt, m->proj, lp.n_in, 2 * hd + 2 * hv, l.w_decay, l.decay_bias, l.tau, m->f32a, NT, l.decay_rank, hd, st));
            RUN(launch_gla_recurrent(dt, m->proj, lp.n_in, m->f32a, (float *)(m->state_pool + lp.state_off), m->f32b, d_start, d_pos0, d_slot, S,
                                     l.heads, l.dim, l.vdim, st, gla_kinds));
            RUN(launch_gla_output(dt, m->f32b, l.out_norm, c.norm_eps, gate, lp.n_in, m->mix2, NT, l.heads, l.vdim, st));
            n_mixed = hv;
        }
        RUN(linear(m, m->mix2, l.w_out, m->y, NT, n_mixed, width, st));
        if (dyt) {
            const float *pre = next_pre(li, 0);
            RUN(residual(true, m->y, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, l.norm, l.post1, l.ls1, pre, trace));
            h_normed = pre != nullptr;
        } else {
            RUN(postnorm(m->y, nullptr, nullptr, 0, nullptr, nullptr, l.norm1, trace));
            h_normed = false;
        }
        if (l.mlp == B200_MLP_NONE) continue;
        trace = layer_trace ? layer_trace + (size_t)li * NT * width : nullptr;
        const void *h2 = dyt ? (const void *)m->h : cast_x();
        const float *pre = next_pre(li, 1);
        const int inner_cols = l.gated ? 2 : 1;
        if (l.mlp == B200_MLP_DENSE) {
            char *up = (char *)m->us, *act = up;
            RUN(linear(m, h2, l.w_up, up, NT, width, inner_cols * l.expert_ff, st));
            if (l.gated) {
                act = up + (size_t)NT * 2 * l.expert_ff * es;
                if (l.b_up) RUN(launch_bias_activation(dt, up, l.b_up, NT, 2 * l.expert_ff, -1, st));
                RUN(launch_gated_activation(dt, up, act, NT, l.expert_ff, l.act, nullptr, 0, st));
            } else {
                RUN(launch_bias_activation(dt, up, l.b_up, NT, l.expert_ff, l.act, st));
            }
            RUN(linear(m, act, l.w_down, m->ys, NT, l.expert_ff, width, st));
            if (dyt) RUN(residual(true, m->ys, l.b_down, nullptr, nullptr, nullptr, 0, nullptr, nullptr, l.norm, l.post2, l.ls2, pre, trace));
            else RUN(residual(true, m->ys, l.b_down, nullptr, nullptr, nullptr, 0, nullptr, nullptr, l.norm, l.norm2, nullptr, nullptr, trace));
            h_normed = dyt && pre != nullptr;
            continue;
        }
        const int pairs = NT * l.top;
        const bool softmax = l.route == B200_ROUTE_SOFTMAX;
        const int outputs = softmax ? l.experts + l.identity : l.experts + 1;
        // prompt-sized batches of a 16-bit engine: 128-row tiles on the tcgen05 grouped GEMM; otherwise 64-row tiles on mma.sync / SIMT
        const bool tc = !f32 && pairs >= 1024 && width % 8 == 0 && l.expert_ff % 8 == 0 && width >= 64 && l.expert_ff >= 64;
        const int tile = tc ? 128 : kMoeTileM;
        const int max_rows = ((pairs + tile - 1) / tile + std::min(l.experts, pairs)) * tile;
        const int max_tiles = max_rows / tile;
        int *sel_expert = m->moe_i, *pair_row = sel_expert + pairs, *row_token = pair_row + pairs, *tile_expert = row_token + max_rows,
            *n_live = tile_expert + max_tiles;
        float *sel_weight = m->moe_f, *row_weight = sel_weight + pairs, *shared_gate = row_weight + max_rows;
        // router logits (+ shared gate), fp32: 16-bit engines multiply the 16-bit copy of the input on the tensor cores (products of 16-bit
        // values are exact in fp32 and the sums are fp32), others -- and widths the tensor-core kernel does not take -- the fp32 kernel
        // (a decode batch is a single 64-row tile there -- one CTA walking all of K -- so few tokens take the fp32 kernel as well)
        rc = NT >= 64 ? launch_dense_f32out(dt, h2, l.w_router, m->f32a, NT, outputs, width, st) : B200_ERR_UNSUPPORTED;
        if (rc == B200_ERR_UNSUPPORTED)
            rc = dyt ? launch_proj_f32(dt, m->h, width, dt, l.w_router, nullptr, m->f32a, outputs, NT, outputs, width, st)
                     : launch_proj_f32(B200_F32, m->x, width, dt, l.w_router, nullptr, m->f32a, outputs, NT, outputs, width, st);
        if (rc != B200_OK) return rc;
        if (softmax) RUN(launch_moe_route_softmax(m->f32a, outputs, l.route_bias, sel_expert, sel_weight, NT, outputs, l.top, st));
        else RUN(launch_moe_route_sigmoid(m->f32a, l.experts + 1, sel_expert, sel_weight, shared_gate, NT, l.experts, l.top, st));
        RUN(launch_moe_plan(sel_expert, sel_weight, row_token, row_weight, tile_expert, pair_row, n_live, NT, l.experts, l.top, tile, st));
        if (softmax) RUN(launch_moe_gather_rows(dt, h2, row_token, m->xg, n_live, max_rows, width, tile, st));
        else RUN(launch_moe_gather(dt, m->x, row_token, row_weight, m->xg, n_live, max_rows, width, tile, st));
        const int n_up = inner_cols * l.expert_ff;
        const int up_act = l.gated ? -1 : l.act;
        char *inner = (char *)m->u;
        if (tc) RUN(launch_gemm_tc_grouped(m->xg, l.w_up, m->u, max_rows, n_up, width, l.experts, tile_expert, n_live, up_act, dt, st));
        else RUN(launch_moe_grouped_gemm(dt, m->xg, l.w_up, m->u, tile_expert, n_live, max_tiles, n_up, width, up_act, st));
        if (l.gated) {
            inner += (size_t)max_rows * n_up * es;
            RUN(launch_gated_activation(dt, m->u, inner, max_rows, l.expert_ff, l.act, n_live, tile, st));
        }
        if (tc) RUN(launch_gemm_tc_grouped(inner, l.w_down, m->yrows, max_rows, width, l.expert_ff, l.experts, tile_expert, n_live, -1, dt, st));
        else RUN(launch_moe_grouped_gemm(dt, inner, l.w_down, m->yrows, tile_expert, n_live, max_tiles, width, l.expert_ff, -1, st));
        if (l.shared_ff > 0) {
            char *sin = (char *)m->us;
            RUN(linear(m, h2, l.w_shared_up, m->us, NT, width, inner_cols * l.shared_ff, st));
            if (l.gated) {
                sin += (size_t)NT * 2 * l.shared_ff * es;
                RUN(launch_gated_activation(dt, m->us, sin, NT, l.shared_ff, l.act, nullptr, 0, st));
            } else {
                RUN(launch_activation(dt, m->us, (size_t)NT * l.shared_ff, l.act, st));
            }
            RUN(linear(m, sin, l.w_shared_down, m->ys, NT, l.shared_ff, width, st));
        }
        const void *y_shared = l.shared_ff > 0 ? m->ys : nullptr;
        if (!softmax) {
            RUN(postnorm(nullptr, m->yrows, pair_row, l.top, y_shared, shared_gate, l.norm2, trace));
            h_normed = false;
        } else {
            RUN(residual(true, nullptr, nullptr, m->yrows, pair_row, sel_weight, l.top, y_shared, nullptr, l.norm, dyt ? l.post2 : l.norm2,
                         dyt ? l.ls2 : nullptr, dyt ? pre : nullptr, trace));
            h_normed = dyt && pre != nullptr;
        }
    }
    if (W > 0) {
        // the wanted rows only: final norm (fp32 and, for 16-bit engines, a 16-bit copy in h), then the LM head with fp32 logits
        B200_DISPATCH_DTYPE(dt, {
            if (c.final_norm == B200_NORM_LN_PARALLEL || c.final_norm == B200_NORM_LN_PRE) final_ln_rows_kernel<T><<<W, 256, 0, st>>>(m->x, d_want, m->final_norm, c.norm_eps, m->xn, f32 ? nullptr : (T *)m->h, width);
            else if (c.final_norm == B200_NORM_DYT_PRE_POST) final_dyt_rows_kernel<T><<<W, 256, 0, st>>>(m->x, d_want, m->final_norm, m->xn, f32 ? nullptr : (T *)m->h, width);
            else final_norm_rows_kernel<T><<<W, 256, 0, st>>>(m->x, d_want, m->final_norm, c.norm_eps, m->xn, f32 ? nullptr : (T *)m->h, width);
        });
        rc = launch_dense_f32out(dt, m->h, m->lm_head, logits, W, c.vocab, width, st);
        if (rc == B200_ERR_UNSUPPORTED) rc = launch_proj_f32(B200_F32, m->xn, width, dt, m->lm_head, nullptr, logits, c.vocab, W, c.vocab, width, st);
        if (rc != B200_OK) return rc;
        const float lscale = c.logit_scale != 0.0f ? c.logit_scale : 1.0f;
        if (c.logit_softcap > 0.0f || lscale != 1.0f) {
            const size_t n = (size_t)W * c.vocab;
            softcap_kernel<<<(unsigned)std::min<size_t>((n + 255) / 256, 148 * 8), 256, 0, st>>>(logits, n, lscale, c.logit_softcap);
        }
    }
#undef RUN
    return cuda_status("hybrid_forward");
}
}
