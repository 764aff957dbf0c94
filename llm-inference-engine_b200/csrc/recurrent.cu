// recurrent.cu -- two recurrent token mixers with an fp32 matrix state per head, for ragged mixed batches (a sequence brings a portion of
// consecutive tokens that continues from its state slot):
//   * gated delta rule (B200_MIXER_DELTA).  q, k, v pass a short causal convolution per channel and silu; q and k become unit vectors per
//     head (q also / sqrt(dim)); per head and key channel a decay g = exp(-exp(a_log) * softplus(W2 z + b)); per head a step beta.
//         S <- diag(g) S;   u = beta * (v - S^T k);   S <- S + k u^T;   o = S^T q
//     then o / rms(o) * w * sigmoid(gate).  The convolutions' last taps - 1 inputs are state as well.
//   * matrix memory with exponential gating (B200_MIXER_MLSTM).  Log gates i, f per head, a running maximum m that starts at 0:
//         m' = max(f + m, i);   S <- exp(f + m - m') S + exp(i - m') k v^T;   n likewise with k alone;
//         o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
//     then o / rms(o) * w * sigmoid(gate).
// Both recurrences are independent per COLUMN of S (one value channel): column_recurrence_kernel gives every column to one thread (or to
// LANES adjacent threads for long key vectors) that keeps it in registers for the whole portion; the per-token key-side vectors are
// staged in shared memory and read as broadcasts.  The normaliser n of the matrix memory is carried as one more column whose value is 1.
// Everything from the projections' outputs on is fp32.
#include "hybrid_ops.cuh"

#include <algorithm>

namespace b200 {

__device__ __forceinline__ float sigmoid_r(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_r(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float logsigmoid_r(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

static int pad4(int n) { return (n + 3) & ~3; }

// fp32 row of one token that the recurrence and the output kernel read.  Every segment starts on a multiple of four floats.
DeltaRow delta_row(int heads, int kv_heads, int dim, int vdim) {
    DeltaRow r;
    r.q = 0, r.k = r.q + pad4(kv_heads * dim), r.v = r.k + pad4(kv_heads * dim), r.decay = r.v + pad4(heads * vdim);
    r.gate = r.decay + pad4(heads * dim), r.beta = r.gate + pad4(heads * vdim), r.ld = r.beta + pad4(heads);
    return r;
}
MlstmRow mlstm_row(int heads, int dim, int vdim) {
    MlstmRow r;
    r.q = 0, r.k = r.q + pad4(heads * dim), r.v = r.k + pad4(heads * dim), r.gi = r.v + pad4(heads * vdim), r.gf = r.gi + pad4(heads);
    r.ld = r.gf + pad4(heads);
    return r;
}

// One CTA per token.  proj row: q | k (kv_heads*dim each) | v (heads*vdim) | step (heads) | decay-in (rank) | gate-in (gate_rank) from col0.
// conv_state: fp32 [slots, taps - 1, channels]: the inputs at positions pos0 - (taps - 1) .. pos0 - 1 of the sequence in that slot.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ conv_w, int taps, const float *__restrict__ conv_state,
                  const T *__restrict__ w_decay, const float *__restrict__ decay_bias, const float *__restrict__ a_log, int rank,
                  const T *__restrict__ w_gate2, int gate_rank, float *__restrict__ rec, DeltaRow lay, const int *__restrict__ tok_seq,
                  const int *__restrict__ tok_pos, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads, int kv_heads, int dim,
                  int vdim) {
    extern __shared__ float sh[];  // conv outputs [channels] | decay-in [rank] | gate-in [gate_rank]
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t], pos0 = seq_pos0[s], slot = seq_slot[s];
    const int nqk = kv_heads * dim, nv = heads * vdim, channels = 2 * nqk + nv;
    float *cv = sh, *zin = cv + channels, *gin = zin + rank;
    const float *cst = conv_state + (size_t)slot * (taps - 1) * channels;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j, pp = pos - back;  // the input `back` tokens ago
            float x = 0.0f;
            if (pp >= pos0) x = Elem<T>::to_f(proj[(size_t)(t - back) * ld + col0 + c]);
            else if (pp >= 0) x = cst[(size_t)(pp - (pos0 - (taps - 1))) * channels + c];
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        cv[c] = acc * sigmoid_r(acc);
    }
    const T *row = proj + (size_t)t * ld + col0 + channels;  // step | decay-in | gate-in
    for (int r = threadIdx.x; r < rank; r += blockDim.x) zin[r] = Elem<T>::to_f(row[heads + r]);
    for (int r = threadIdx.x; r < gate_rank; r += blockDim.x) gin[r] = Elem<T>::to_f(row[heads + rank + r]);
    __syncthreads();
    float *out = rec + (size_t)t * lay.ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int hh = warp; hh < 2 * kv_heads; hh += nwarp) {  // unit vectors: q heads, then k heads
        const float *src = cv + hh * dim;
        float ss = 0.0f;
        for (int c = lane; c < dim; c += 32) ss = fmaf(src[c], src[c], ss);
        const bool is_q = hh < kv_heads;
        const float inv = rsqrtf(warp_sum(ss) + 1e-6f) * (is_q ? rsqrtf((float)dim) : 1.0f);
        float *dst = out + (is_q ? lay.q + hh * dim : lay.k + (hh - kv_heads) * dim);
        for (int c = lane; c < dim; c += 32) dst[c] = src[c] * inv;
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) out[lay.v + c] = cv[2 * nqk + c];
    for (int h = threadIdx.x; h < heads; h += blockDim.x) out[lay.beta + h] = sigmoid_r(Elem<T>::to_f(row[h]));
    for (int c = threadIdx.x; c < heads * dim; c += blockDim.x) {
        float z = decay_bias ? decay_bias[c] : 0.0f;
        const T *wr = w_decay + (size_t)c * rank;
        for (int r = 0; r < rank; ++r) z = fmaf(Elem<T>::to_f(wr[r]), zin[r], z);
        out[lay.decay + c] = expf(-expf(a_log[c / dim]) * softplus_r(z));
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        float z = 0.0f;
        const T *wr = w_gate2 + (size_t)c * gate_rank;
        for (int r = 0; r < gate_rank; ++r) z = fmaf(Elem<T>::to_f(wr[r]), gin[r], z);
        out[lay.gate + c] = z;  // the output kernel applies the sigmoid
    }
}

// After the convolutions have read it: the state's rows move up by the portion's length and its last inputs come in.  One CTA per
// sequence; a thread owns whole channels, so it reads what it overwrites before it does.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T *__restrict__ proj, int ld, int col0, float *__restrict__ conv_state, int taps, int channels,
                         const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot) {
    const int s = blockIdx.x, t0 = seq_start[s], len = seq_start[s + 1] - t0, pos0 = seq_pos0[s], keep = taps - 1;
    if (len <= 0) return;
    float *cst = conv_state + (size_t)seq_slot[s] * keep * channels;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        for (int r = 0; r < keep; ++r) {  // new row r holds the input at position pos0 + len - keep + r; ascending r reads rows >= r only
            const int i = len - keep + r;  // index into the portion
            float x = 0.0f;
            if (i >= 0) x = Elem<T>::to_f(proj[(size_t)(t0 + i) * ld + col0 + c]);
            else if (pos0 + i >= 0) x = cst[(size_t)(r + len) * channels + c];
            cst[(size_t)r * channels + c] = x;
        }
    }
}

// proj row: q | k (heads*dim each) | v | gate (heads*vdim each) | input gate | forget gate (heads each) from col0; b_in (optional) the same.
template <typename T>
__global__ void __launch_bounds__(256)
mlstm_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ b_in, float cap, float *__restrict__ rec, MlstmRow lay,
                  int heads, int dim, int vdim) {
    const int t = blockIdx.x;
    const T *row = proj + (size_t)t * ld + col0;
    const float *bias = b_in;  // counted from the mixer's own first row
    float *out = rec + (size_t)t * lay.ld;
    const int nqk = heads * dim, nv = heads * vdim;
    const float qs = rsqrtf((float)dim);
    for (int c = threadIdx.x; c < nqk; c += blockDim.x) {
        out[lay.q + c] = (Elem<T>::to_f(row[c]) + (bias ? bias[c] : 0.0f)) * qs;
        out[lay.k + c] = Elem<T>::to_f(row[nqk + c]) + (bias ? bias[nqk + c] : 0.0f);
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) out[lay.v + c] = Elem<T>::to_f(row[2 * nqk + c]) + (bias ? bias[2 * nqk + c] : 0.0f);
    const int g0 = 2 * nqk + 2 * nv;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float zi = Elem<T>::to_f(row[g0 + h]) + (bias ? bias[g0 + h] : 0.0f);
        const float zf = Elem<T>::to_f(row[g0 + heads + h]) + (bias ? bias[g0 + heads + h] : 0.0f);
        out[lay.gi + h] = cap > 0.0f ? cap * tanhf(zi / cap) : zi;
        out[lay.gf + h] = logsigmoid_r(cap > 0.0f ? cap * tanhf(zf / cap) : zf);
    }
}

// grid (column tiles, heads, sequences); blockDim = CB * LANES threads.  A column's rows r = sub * RPT + i live in registers of lane `sub`.
// MODE 0 (delta): per token k, q, decay [dim] and beta;  MODE 1 (matrix memory): per token k, q [dim] and the log gates.
// Shared memory per staged token: kq[3 * DP] (k | q | decay, DP = RPT * LANES, zero beyond dim) | two scalars; kTB tokens per stage.
constexpr int kRecTB = 8;

template <int RPT, int LANES, int MODE>
__global__ void __launch_bounds__(128)
column_recurrence_kernel(const float *__restrict__ rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off,
                         float *__restrict__ S, float *__restrict__ n_state, float *__restrict__ m_state, float *__restrict__ o,
                         float *__restrict__ nq_out, float *__restrict__ m_out, const int *__restrict__ seq_start,
                         const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads, int kv_heads, int dim, int vdim) {
    constexpr int DP = RPT * LANES, NV = MODE == 0 ? 3 : 2;
    extern __shared__ __align__(16) float stage[];  // [kRecTB][NV * DP + 4] | v [kRecTB][CB]
    const int CB = blockDim.x / LANES;
    constexpr int TS = NV * DP + 4;
    float *vs = stage + kRecTB * TS;
    const int s = blockIdx.z, h = blockIdx.y, g = h / (heads / kv_heads);
    const int t0 = seq_start[s], len = seq_start[s + 1] - t0;
    if (len <= 0) return;
    const int pos0 = seq_pos0[s], slot = seq_slot[s];
    const int ncols = MODE == 1 ? vdim + 1 : vdim;
    const int cl = threadIdx.x / LANES, sub = threadIdx.x % LANES;
    const int col = blockIdx.x * CB + cl;
    const bool active = col < ncols, is_n = MODE == 1 && col == vdim;
    const int r0 = sub * RPT;
    float *Sp = S + ((size_t)slot * heads + h) * dim * vdim;
    float *np = MODE == 1 ? n_state + ((size_t)slot * heads + h) * dim : nullptr;

    float st[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = r0 + i;
        st[i] = (pos0 > 0 && active && r < dim) ? (is_n ? np[r] : Sp[(size_t)r * vdim + col]) : 0.0f;
    }
    float m = (MODE == 1 && pos0 > 0) ? m_state[(size_t)slot * heads + h] : 0.0f;

    for (int c0 = 0; c0 < len; c0 += kRecTB) {
        const int nt = min(kRecTB, len - c0);
        __syncthreads();  // the previous stage has been consumed
        for (int i = threadIdx.x; i < nt * NV * DP; i += blockDim.x) {
            const int tt = i / (NV * DP), w = i - tt * (NV * DP), which = w / DP, r = w - which * DP;
            const float *row = rec + (size_t)(t0 + c0 + tt) * rec_ld;
            float x = 0.0f;
            if (r < dim) x = which == 0 ? row[k_off + g * dim + r] : (which == 1 ? row[q_off + g * dim + r] : row[a_off + h * dim + r]);
            stage[tt * TS + w] = x;
        }
        for (int i = threadIdx.x; i < nt * 2; i += blockDim.x) {
            const int tt = i >> 1, w = i & 1;
            const float *row = rec + (size_t)(t0 + c0 + tt) * rec_ld;
            stage[tt * TS + NV * DP + w] = MODE == 0 ? row[b_off + h] : (w == 0 ? row[a_off + h] : row[b_off + h]);
        }
        for (int i = threadIdx.x; i < nt * CB; i += blockDim.x) {
            const int tt = i / CB, c = blockIdx.x * CB + (i - tt * CB);
            vs[tt * CB + (i - tt * CB)] = c < vdim ? rec[(size_t)(t0 + c0 + tt) * rec_ld + v_off + h * vdim + c] : 1.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float4 *kp = reinterpret_cast<const float4 *>(stage + tt * TS + r0);
            const float4 *qp = reinterpret_cast<const float4 *>(stage + tt * TS + DP + r0);
            const float v = vs[tt * CB + cl];
            float out0 = 0.0f, out1 = 0.0f;
            if (MODE == 0) {
                const float4 *gp = reinterpret_cast<const float4 *>(stage + tt * TS + 2 * DP + r0);
                const float beta = stage[tt * TS + NV * DP];
                float d0 = 0.0f, d1 = 0.0f;
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 kk = kp[i >> 2], gg = gp[i >> 2];
                    st[i] *= gg.x, st[i + 1] *= gg.y, st[i + 2] *= gg.z, st[i + 3] *= gg.w;
                    d0 = fmaf(kk.x, st[i], d0), d1 = fmaf(kk.y, st[i + 1], d1), d0 = fmaf(kk.z, st[i + 2], d0), d1 = fmaf(kk.w, st[i + 3], d1);
                }
                float dot = d0 + d1;
#pragma unroll
                for (int w = LANES >> 1; w > 0; w >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, w);
                const float u = beta * (v - dot);
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 kk = kp[i >> 2], qq = qp[i >> 2];
                    st[i] = fmaf(kk.x, u, st[i]), st[i + 1] = fmaf(kk.y, u, st[i + 1]), st[i + 2] = fmaf(kk.z, u, st[i + 2]), st[i + 3] = fmaf(kk.w, u, st[i + 3]);
                    out0 = fmaf(qq.x, st[i], out0), out1 = fmaf(qq.y, st[i + 1], out1), out0 = fmaf(qq.z, st[i + 2], out0), out1 = fmaf(qq.w, st[i + 3], out1);
                }
            } else {
                const float gi = stage[tt * TS + NV * DP], gf = stage[tt * TS + NV * DP + 1];
                const float m_new = fmaxf(gf + m, gi);
                const float a = expf(gf + m - m_new), bv = expf(gi - m_new) * v;
                m = m_new;
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 kk = kp[i >> 2], qq = qp[i >> 2];
                    st[i] = fmaf(a, st[i], kk.x * bv), st[i + 1] = fmaf(a, st[i + 1], kk.y * bv), st[i + 2] = fmaf(a, st[i + 2], kk.z * bv), st[i + 3] = fmaf(a, st[i + 3], kk.w * bv);
                    out0 = fmaf(qq.x, st[i], out0), out1 = fmaf(qq.y, st[i + 1], out1), out0 = fmaf(qq.z, st[i + 2], out0), out1 = fmaf(qq.w, st[i + 3], out1);
                }
            }
            float out = out0 + out1;
#pragma unroll
            for (int w = LANES >> 1; w > 0; w >>= 1) out += __shfl_xor_sync(0xffffffffu, out, w);
            if (active && sub == 0) {
                const size_t tok = (size_t)(t0 + c0 + tt);
                if (is_n) nq_out[tok * heads + h] = out, m_out[tok * heads + h] = m;
                else o[(tok * heads + h) * vdim + col] = out;
            }
        }
    }
    if (!active) return;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = r0 + i;
        if (r < dim) {
            if (is_n) np[r] = st[i];
            else Sp[(size_t)r * vdim + col] = st[i];
        }
    }
    if (is_n && sub == 0) m_state[(size_t)slot * heads + h] = m;
}

// One warp per (token, head): out[t, h*vdim + j] = out_scale * y_j * rsqrt(mean_j y^2 + eps) * w[h * w_stride + j] * sigmoid(gate),
// y = o (delta) or o / (max(|nq|, exp(-m)) + 1e-6) (matrix memory: nq != NULL).  gate: fp32 pre-activations (gate_f) or the projection's.
template <typename T>
__global__ void __launch_bounds__(256)
head_output_kernel(const float *__restrict__ o, const float *__restrict__ nq, const float *__restrict__ m_in, const float *__restrict__ w,
                   int w_stride, float eps, const float *__restrict__ gate_f, int gate_f_ld, const T *__restrict__ gate_t, int gate_t_ld,
                   T *__restrict__ out, int out_ld, float out_scale, int tokens, int heads, int vdim) {
    const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (idx >= tokens * heads) return;
    const int t = idx / heads, h = idx - t * heads;
    const float *src = o + (size_t)idx * vdim;
    float inv_den = 1.0f;
    if (nq) inv_den = 1.0f / (fmaxf(fabsf(nq[idx]), expf(-m_in[idx])) + 1e-6f);
    float ss = 0.0f;
    for (int j = lane; j < vdim; j += 32) {
        const float y = src[j] * inv_den;
        ss = fmaf(y, y, ss);
    }
    const float inv = rsqrtf(warp_sum(ss) / (float)vdim + eps) * inv_den;
    for (int j = lane; j < vdim; j += 32) {
        const float z = gate_f ? gate_f[(size_t)t * gate_f_ld + h * vdim + j] : Elem<T>::to_f(gate_t[(size_t)t * gate_t_ld + h * vdim + j]);
        out[(size_t)t * out_ld + h * vdim + j] = Elem<T>::from_f(src[j] * inv * w[h * w_stride + j] * sigmoid_r(z) * out_scale);
    }
}

template <int RPT, int LANES, int MODE>
static int launch_colrec_t(const float *rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off, float *S, float *n_state,
                           float *m_state, float *o, float *nq, float *m_out, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                           int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t st) {
    const int ncols = MODE == 1 ? vdim + 1 : vdim;
    // few sequences: narrow column tiles spread a portion's columns over more SMs
    int cb = 128 / LANES;
    while (cb > 32 / LANES && cb > 8 && (long long)((ncols + cb - 1) / cb) * heads * n_seqs < 2 * 148) cb >>= 1;
    if (cb * LANES < 32) cb = 32 / LANES;
    constexpr int NV = MODE == 0 ? 3 : 2;
    const size_t smem = ((size_t)kRecTB * (NV * RPT * LANES + 4) + (size_t)kRecTB * cb) * sizeof(float);
    auto kern = column_recurrence_kernel<RPT, LANES, MODE>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<dim3((ncols + cb - 1) / cb, heads, n_seqs), cb * LANES, smem, st>>>(rec, rec_ld, q_off, k_off, v_off, a_off, b_off, S, n_state, m_state, o, nq,
                                                                             m_out, seq_start, seq_pos0, seq_slot, heads, kv_heads, dim, vdim);
    return cuda_status("column_recurrence launch");
}

template <int MODE>
static int launch_colrec(const float *rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off, float *S, float *n_state,
                         float *m_state, float *o, float *nq, float *m_out, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                         int n_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t st) {
    if (n_seqs == 0) return B200_OK;
#define B200_COLREC(R, L) \
    return launch_colrec_t<R, L, MODE>(rec, rec_ld, q_off, k_off, v_off, a_off, b_off, S, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot, n_seqs, heads, kv_heads, dim, vdim, st)
    if (dim <= 16) B200_COLREC(16, 1);
    if (dim <= 32) B200_COLREC(32, 1);
    if (dim <= 48) B200_COLREC(48, 1);
    if (dim <= 64) B200_COLREC(64, 1);
    if (dim <= 96) B200_COLREC(96, 1);
    if (dim <= 128) B200_COLREC(128, 1);
    if (dim <= 256) B200_COLREC(128, 2);
    if (dim <= 512) B200_COLREC(128, 4);
#undef B200_COLREC
    set_error("column recurrence: key size %d above 512", dim);
    return B200_ERR_UNSUPPORTED;
}

int launch_delta_prep(int dtype, const void *proj, int ld, int col0, const float *conv_w, int taps, float *conv_state, const void *w_decay,
                      const float *decay_bias, const float *a_log, int rank, const void *w_gate2, int gate_rank, float *rec, const int *tok_seq,
                      const int *tok_pos, const int *seq_start, const int *seq_pos0, const int *seq_slot, int tokens, int heads, int kv_heads,
                      int dim, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const DeltaRow lay = delta_row(heads, kv_heads, dim, vdim);
    const size_t smem = ((size_t)2 * kv_heads * dim + heads * vdim + rank + gate_rank) * sizeof(float);
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        delta_prep_kernel<T><<<tokens, 256, smem, st>>>((const T *)proj, ld, col0, conv_w, taps, conv_state, (const T *)w_decay, decay_bias, a_log, rank,
                                                       (const T *)w_gate2, gate_rank, rec, lay, tok_seq, tok_pos, seq_pos0, seq_slot, heads, kv_heads, dim,
                                                       vdim);
    });
    return cuda_status("delta_prep launch");
}

int launch_conv_state_update(int dtype, const void *proj, int ld, int col0, float *conv_state, int taps, int channels, const int *seq_start,
                             const int *seq_pos0, const int *seq_slot, int n_seqs, cudaStream_t st) {
    if (n_seqs == 0 || taps <= 1) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        conv_state_update_kernel<T><<<n_seqs, 256, 0, st>>>((const T *)proj, ld, col0, conv_state, taps, channels, seq_start, seq_pos0, seq_slot);
    });
    return cuda_status("conv_state_update launch");
}

int launch_delta_recurrent(const float *rec, float *S, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs,
                           int heads, int kv_heads, int dim, int vdim, cudaStream_t st) {
    const DeltaRow lay = delta_row(heads, kv_heads, dim, vdim);
    return launch_colrec<0>(rec, lay.ld, lay.q, lay.k, lay.v, lay.decay, lay.beta, S, nullptr, nullptr, o, nullptr, nullptr, seq_start, seq_pos0,
                            seq_slot, n_seqs, heads, kv_heads, dim, vdim, st);
}

int launch_mlstm_prep(int dtype, const void *proj, int ld, int col0, const float *b_in, float cap, float *rec, int tokens, int heads, int dim,
                      int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const MlstmRow lay = mlstm_row(heads, dim, vdim);
    B200_DISPATCH_DTYPE(dtype, { mlstm_prep_kernel<T><<<tokens, 256, 0, st>>>((const T *)proj, ld, col0, b_in, cap, rec, lay, heads, dim, vdim); });
    return cuda_status("mlstm_prep launch");
}

int launch_mlstm_recurrent(const float *rec, float *S, float *n_state, float *m_state, float *o, float *nq, float *m_out, const int *seq_start,
                           const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st) {
    const MlstmRow lay = mlstm_row(heads, dim, vdim);
    return launch_colrec<1>(rec, lay.ld, lay.q, lay.k, lay.v, lay.gi, lay.gf, S, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot,
                            n_seqs, heads, heads, dim, vdim, st);
}

int launch_head_output(int dtype, const float *o, const float *nq, const float *m_in, const float *w, int w_stride, float eps,
                       const float *gate_f, int gate_f_ld, const void *gate_t, int gate_t_ld, void *out, int out_ld, float out_scale, int tokens,
                       int heads, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const int grid = (tokens * heads + 7) / 8;
    B200_DISPATCH_DTYPE(dtype, {
        head_output_kernel<T><<<grid, 256, 0, st>>>(o, nq, m_in, w, w_stride, eps, gate_f, gate_f_ld, (const T *)gate_t, gate_t_ld, (T *)out, out_ld,
                                                   out_scale, tokens, heads, vdim);
    });
    return cuda_status("head_output launch");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_delta_rule_recurrent(const float *rec, float *state, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                              int n_seqs, int heads, int kv_heads, int dim, int vdim, b200_stream_t stream) {
    B200_REQUIRE(rec && state && o && seq_start && seq_pos0 && seq_slot, "delta_rule_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "delta_rule_recurrent: bad shape");
    return launch_delta_recurrent(rec, state, o, seq_start, seq_pos0, seq_slot, n_seqs, heads, kv_heads, dim, vdim, as_stream(stream));
}

int b200_mlstm_recurrent(const float *rec, float *state, float *n_state, float *m_state, float *o, float *nq, float *m_out,
                         const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim,
                         b200_stream_t stream) {
    B200_REQUIRE(rec && state && n_state && m_state && o && nq && m_out && seq_start && seq_pos0 && seq_slot, "mlstm_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, "mlstm_recurrent: bad shape");
    return launch_mlstm_recurrent(rec, state, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot, n_seqs, heads, dim, vdim,
                                  as_stream(stream));
}
}
