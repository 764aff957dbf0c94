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
//   * decayed outer-product memory with ONE decay per head and token:  S <- a S + k v^T;  o = S^T q.  Two mixers are this recurrence
//     behind different prep steps: the state-space mixer (B200_MIXER_SSD: convolution + silu on x | B | C, step size dt = softplus(z + b),
//     a = exp(-exp(a_log) dt), k = B, v = dt x, q = C, plus a skip term) and linear attention with a constant decay per head
//     (B200_MIXER_LINEAR: q, k, v = silu of their projections).  The gated delta rule with one decay per head and full-rank gates takes
//     delta_prep_direct_kernel and the delta recurrence.
// All recurrences are independent per COLUMN of S (one value channel): column_recurrence_kernel gives every column to one thread (or to
// LANES adjacent threads for long key vectors) that keeps it in registers for the whole portion; the per-token key-side vectors are
// staged in shared memory and read as broadcasts.  The normaliser n of the matrix memory is carried as one more column whose value is 1.
// Everything from the projections' outputs on is fp32.
#include "hybrid_ops.cuh"

#include <algorithm>
#include <cstdlib>

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
DecayRow decay_row(int heads, int kv_heads, int dim, int vdim) {
    DecayRow r;
    r.q = 0, r.k = r.q + pad4(kv_heads * dim), r.v = r.k + pad4(kv_heads * dim), r.skip = r.v + pad4(heads * vdim);
    r.decay = r.skip + pad4(heads * vdim), r.ld = r.decay + pad4(heads);
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
// Writes q, k (unit vectors), v and the step of the token's fp32 row, and the two low-rank inputs as dense rows lr_a [tokens, rank],
// lr_g [tokens, gate_rank] for the products that follow.
template <typename T>
__global__ void __launch_bounds__(1024)
delta_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ conv_w, int taps, const float *__restrict__ conv_state,
                  int rank, int gate_rank, T *__restrict__ lr_a, T *__restrict__ lr_g, float *__restrict__ rec, DeltaRow lay,
                  const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ seq_pos0,
                  const int *__restrict__ seq_slot, int heads, int kv_heads, int dim, int vdim) {
    extern __shared__ float sh[];  // conv outputs [channels]
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t], pos0 = seq_pos0[s], slot = seq_slot[s];
    const int nqk = kv_heads * dim, nv = heads * vdim, channels = 2 * nqk + nv;
    float *cv = sh;
    const float *cst = conv_state + (size_t)slot * (taps - 1) * channels;
    // every tap reads both places it could come from at an index that always exists and keeps the one that is meant: no branch stands
    // between the loads, so the taps' (and, unrolled, four channels') loads are in flight together
    const int keep = taps > 1 ? taps - 1 : 1;
#pragma unroll 4
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j, pp = pos - back;  // the input `back` tokens ago
            const float xp = Elem<T>::to_f(proj[(size_t)max(t - back, 0) * ld + col0 + c]);
            const float xs = cst[(size_t)min(max(pp - (pos0 - (taps - 1)), 0), keep - 1) * channels + c];
            const float x = pp >= pos0 ? xp : (pp >= 0 ? xs : 0.0f);
            acc = fmaf(conv_w[(size_t)c * taps + j], x, acc);
        }
        cv[c] = acc * sigmoid_r(acc);
    }
    const T *row = proj + (size_t)t * ld + col0 + channels;  // step | decay-in | gate-in
    for (int r = threadIdx.x; r < rank; r += blockDim.x) lr_a[(size_t)t * rank + r] = row[heads + r];
    for (int r = threadIdx.x; r < gate_rank; r += blockDim.x) lr_g[(size_t)t * gate_rank + r] = row[heads + rank + r];
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
}

// The causal convolution of channel c at token t (packed row) / position pos: taps - 1 earlier inputs come from the portion's own rows,
// from the slot's stored inputs (positions before pos0) or are zero (before position 0).  Every tap reads both places at an index that
// always exists and keeps the one that is meant.
template <typename T>
__device__ __forceinline__ float conv_at(const T *__restrict__ proj, int ld, int col, int t, int pos, int pos0, const float *__restrict__ w, int taps,
                                         const float *__restrict__ cst, int channels, int c) {
    const int keep = taps > 1 ? taps - 1 : 1;
    float acc = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int back = taps - 1 - j, pp = pos - back;
        const float xp = Elem<T>::to_f(proj[(size_t)max(t - back, 0) * ld + col + c]);
        const float xs = cst[(size_t)min(max(pp - (pos0 - (taps - 1)), 0), keep - 1) * channels + c];
        const float x = pp >= pos0 ? xp : (pp >= 0 ? xs : 0.0f);
        acc = fmaf(w[(size_t)c * taps + j], x, acc);
    }
    return acc;
}

// The delta rule with full-rank gates and one decay per head.  proj row from col0: q | k (kv_heads*dim each) | v (heads*vdim) | step
// (heads) | decay-in (heads) | gate (heads*vdim; read by the output kernel).  Writes q, k (unit vectors), v, the step and the decay
// exp(-exp(a_log[h]) * softplus(decay-in[h] + bias[h])), repeated over the head's key channels, into the token's fp32 row.
template <typename T>
__global__ void __launch_bounds__(1024)
delta_prep_direct_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ conv_w, int taps, const float *__restrict__ conv_state,
                         const float *__restrict__ decay_bias, const float *__restrict__ a_log, float *__restrict__ rec, DeltaRow lay,
                         const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ seq_pos0,
                         const int *__restrict__ seq_slot, int heads, int kv_heads, int dim, int vdim) {
    extern __shared__ float sh[];  // conv outputs [channels]
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t], pos0 = seq_pos0[s], slot = seq_slot[s];
    const int nqk = kv_heads * dim, nv = heads * vdim, channels = 2 * nqk + nv;
    const float *cst = conv_state + (size_t)slot * (taps - 1) * channels;
#pragma unroll 4
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        const float acc = conv_at<T>(proj, ld, col0, t, pos, pos0, conv_w, taps, cst, channels, c);
        sh[c] = acc * sigmoid_r(acc);
    }
    __syncthreads();
    const T *row = proj + (size_t)t * ld + col0 + channels;  // step | decay-in | gate
    float *out = rec + (size_t)t * lay.ld;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int hh = warp; hh < 2 * kv_heads; hh += nwarp) {  // unit vectors: q heads, then k heads
        const float *src = sh + hh * dim;
        float ss = 0.0f;
        for (int c = lane; c < dim; c += 32) ss = fmaf(src[c], src[c], ss);
        const bool is_q = hh < kv_heads;
        const float inv = rsqrtf(warp_sum(ss) + 1e-6f) * (is_q ? rsqrtf((float)dim) : 1.0f);
        float *dst = out + (is_q ? lay.q + hh * dim : lay.k + (hh - kv_heads) * dim);
        for (int c = lane; c < dim; c += 32) dst[c] = src[c] * inv;
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) out[lay.v + c] = sh[2 * nqk + c];
    for (int h = threadIdx.x; h < heads; h += blockDim.x) out[lay.beta + h] = sigmoid_r(Elem<T>::to_f(row[h]));
    for (int c = threadIdx.x; c < heads * dim; c += blockDim.x) {
        const int h = c / dim;
        const float z = Elem<T>::to_f(row[heads + h]) + (decay_bias ? decay_bias[h] : 0.0f);
        out[lay.decay + c] = expf(-expf(a_log[h]) * softplus_r(z));
    }
}

// The state-space mixer's prep.  proj row from col0: z | x (heads*vdim each) | B | C (groups*state each) | dt (heads).  x | B | C pass the
// convolution (+ bias) and silu.  Writes the token's fp32 row: q = C, k = B, v = dt * x, skip = skip_w[h] * x, decay = exp(-exp(a_log) dt),
// dt = softplus(dt-in + dt_bias), unclamped.
template <typename T>
__global__ void __launch_bounds__(1024)
ssd_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ conv_w, const float *__restrict__ conv_b, int taps,
                const float *__restrict__ conv_state, const float *__restrict__ dt_bias, const float *__restrict__ a_log,
                const float *__restrict__ skip_w, float *__restrict__ rec, DecayRow lay, const int *__restrict__ tok_seq,
                const int *__restrict__ tok_pos, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads, int groups,
                int state, int vdim) {
    extern __shared__ float sh[];  // dt [heads]
    const int t = blockIdx.x, s = tok_seq[t], pos = tok_pos[t], pos0 = seq_pos0[s], slot = seq_slot[s];
    const int inner = heads * vdim, gn = groups * state, channels = inner + 2 * gn;
    const float *cst = conv_state + (size_t)slot * (taps - 1) * channels;
    const T *row = proj + (size_t)t * ld + col0;
    float *out = rec + (size_t)t * lay.ld;
    for (int h = threadIdx.x; h < heads; h += blockDim.x) {
        const float dt = softplus_r(Elem<T>::to_f(row[2 * inner + 2 * gn + h]) + (dt_bias ? dt_bias[h] : 0.0f));
        sh[h] = dt;
        out[lay.decay + h] = expf(-expf(a_log[h]) * dt);
    }
    __syncthreads();
#pragma unroll 4
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = conv_at<T>(proj, ld, col0 + inner, t, pos, pos0, conv_w, taps, cst, channels, c);
        if (conv_b) acc += conv_b[c];
        const float v = acc * sigmoid_r(acc);
        if (c < inner) {
            const int h = c / vdim;
            out[lay.v + c] = sh[h] * v;
            out[lay.skip + c] = skip_w ? skip_w[h] * v : 0.0f;
        } else if (c < inner + gn) {
            out[lay.k + (c - inner)] = v;
        } else {
            out[lay.q + (c - inner - gn)] = v;
        }
    }
}

// Linear attention with a constant decay per head.  proj row from col0: q | k (heads*dim each) | v | gate (heads*vdim each).
template <typename T>
__global__ void __launch_bounds__(256)
linear_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ head_decay, float *__restrict__ rec, DecayRow lay,
                   int heads, int dim, int vdim) {
    const int t = blockIdx.x, nqk = heads * dim, nv = heads * vdim;
    const T *row = proj + (size_t)t * ld + col0;
    float *out = rec + (size_t)t * lay.ld;
    for (int c = threadIdx.x; c < nqk; c += blockDim.x) {
        const float q = Elem<T>::to_f(row[c]), k = Elem<T>::to_f(row[nqk + c]);
        out[lay.q + c] = q * sigmoid_r(q);
        out[lay.k + c] = k * sigmoid_r(k);
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) {
        const float v = Elem<T>::to_f(row[2 * nqk + c]);
        out[lay.v + c] = v * sigmoid_r(v);
    }
    for (int h = threadIdx.x; h < heads; h += blockDim.x) out[lay.decay + h] = head_decay[h];
}

// One CTA per (token, group): the read-out of a whole token (or of one of `groups` equal parts of it) normed together.
//   y_c = o[t, c] + skip[t * skip_ld + c];   gate_first: y_c *= act(gate_c);   out[t, c] = T(y_c * rsqrt(mean_c y^2 + eps) * w[c] * (gate_first
//   ? 1 : act(gate_c))), act = silu (gate_act 1) or sigmoid (0); c runs over the group's columns of the row of `cols`.
// VEC: four columns per access (every piece starts on a boundary of its access).  A thread's values stay in registers between the sum and
// the scaling when the group is short enough (kKeep pieces per thread), else they are formed twice.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
group_output_kernel(const float *__restrict__ o, const float *__restrict__ skip, int skip_ld, const float *__restrict__ w, float eps,
                    const T *__restrict__ gate, int gate_ld, int gate_act, int gate_first, T *__restrict__ out, int out_ld, int cols, int groups) {
    __shared__ float red[33];
    constexpr int N = VEC ? 4 : 1, kKeep = VEC ? 2 : 8;
    const int t = blockIdx.x / groups, g = blockIdx.x - t * groups, per = cols / groups, c0 = g * per;
    auto act = [&](float z) { return gate_act ? z * sigmoid_r(z) : sigmoid_r(z); };
    auto value = [&](int c, float *y) {
        load_n<float, N>(o + (size_t)t * cols + c, y);
        if (skip) {
            float sk[N];
            load_n<float, N>(skip + (size_t)t * skip_ld + c, sk);
#pragma unroll
            for (int i = 0; i < N; ++i) y[i] += sk[i];
        }
        if (gate_first) {
            float z[N];
            load_n<T, N>(gate + (size_t)t * gate_ld + c, z);
#pragma unroll
            for (int i = 0; i < N; ++i) y[i] *= act(z[i]);
        }
    };
    auto finish = [&](int c, float *y, float inv) {
        float wv[N];
        load_n<float, N>(w + c, wv);
#pragma unroll
        for (int i = 0; i < N; ++i) y[i] *= inv * wv[i];
        if (!gate_first) {
            float z[N];
            load_n<T, N>(gate + (size_t)t * gate_ld + c, z);
#pragma unroll
            for (int i = 0; i < N; ++i) y[i] *= act(z[i]);
        }
        store_n<T, N>(out + (size_t)t * out_ld + c, y);
    };
    const bool keep = per <= (int)blockDim.x * kKeep * N;
    float held[kKeep][N];
    float ss = 0.0f;
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = c0 + (threadIdx.x + i * blockDim.x) * N;
            if (c < c0 + per) {
                value(c, held[i]);
#pragma unroll
                for (int e = 0; e < N; ++e) ss = fmaf(held[i][e], held[i][e], ss);
            }
        }
    } else {
        for (int c = c0 + threadIdx.x * N; c < c0 + per; c += blockDim.x * N) {
            float y[N];
            value(c, y);
#pragma unroll
            for (int e = 0; e < N; ++e) ss = fmaf(y[e], y[e], ss);
        }
    }
    const float inv = rsqrtf(block_sum(ss, red) / (float)per + eps);
    if (keep) {
#pragma unroll
        for (int i = 0; i < kKeep; ++i) {
            const int c = c0 + (threadIdx.x + i * blockDim.x) * N;
            if (c < c0 + per) finish(c, held[i], inv);
        }
        return;
    }
    for (int c = c0 + threadIdx.x * N; c < c0 + per; c += blockDim.x * N) {
        float y[N];
        value(c, y);
        finish(c, y, inv);
    }
}

// za fp32 [tokens, heads*dim] = w_decay . decay-in, zg fp32 [tokens, heads*vdim] = w_gate2 . gate-in (the products of the two low-rank
// inputs) -> the token row's decay = exp(-exp(a_log[head]) * softplus(za + bias)) and gate pre-activation (the output kernel applies
// the sigmoid)
__global__ void __launch_bounds__(256)
delta_finish_kernel(const float *__restrict__ za, const float *__restrict__ zg, const float *__restrict__ decay_bias, const float *__restrict__ a_log,
                    float *__restrict__ rec, DeltaRow lay, int heads, int dim, int vdim) {
    const int t = blockIdx.x, nd = heads * dim, nv = heads * vdim;
    float *out = rec + (size_t)t * lay.ld;
    for (int c = threadIdx.x; c < nd; c += blockDim.x) {
        const float z = za[(size_t)t * nd + c] + (decay_bias ? decay_bias[c] : 0.0f);
        out[lay.decay + c] = expf(-expf(a_log[c / dim]) * softplus_r(z));
    }
    for (int c = threadIdx.x; c < nv; c += blockDim.x) out[lay.gate + c] = zg[(size_t)t * nv + c];
}

// After the convolutions have read it: the state's rows move up by the portion's length and its last inputs come in.  grid (channel
// blocks, sequences); a thread owns a whole channel, so it reads what it overwrites before it does.
template <typename T>
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const T *__restrict__ proj, int ld, int col0, float *__restrict__ conv_state, int taps, int channels,
                         const int *__restrict__ seq_start, const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot) {
    const int s = blockIdx.y, t0 = seq_start[s], len = seq_start[s + 1] - t0, pos0 = seq_pos0[s], keep = taps - 1;
    if (len <= 0) return;
    float *cst = conv_state + (size_t)seq_slot[s] * keep * channels;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < channels; c += gridDim.x * blockDim.x) {
        for (int r = 0; r < keep; ++r) {  // new row r holds the input at position pos0 + len - keep + r; ascending r reads rows >= r only
            const int i = len - keep + r;  // index into the portion
            const float xp = Elem<T>::to_f(proj[(size_t)(t0 + max(i, 0)) * ld + col0 + c]);
            const float xs = cst[(size_t)min(r + len, keep - 1) * channels + c];
            cst[(size_t)r * channels + c] = i >= 0 ? xp : (pos0 + i >= 0 ? xs : 0.0f);
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

// grid (column tiles, heads, sequences); blockDim = CB / CPT * LANES threads.  A thread holds a tile of the state in registers: CPT adjacent
// columns x RPT = DP / LANES rows, the rows dealt out over the LANES adjacent threads of a column group in fours (lane `sub` holds rows
// 4 * (sub + LANES * j) .. + 3, so the lanes read consecutive 16-byte pieces of a staged vector: no bank conflicts).  A staged key-side value
// is read once for the thread's CPT columns, the columns' chains run side by side, and dot products over the rows end in a butterfly over
// the lanes.  The host picks LANES by how many columns the batch has: one long prompt spreads every column group over many threads (the
// token loop is sequential, its length per token is RPT), a decode batch of many sequences keeps longer pieces of a column in one thread.
// MODE 0 (delta): per token k, q, decay [dim] and the step;  MODE 1 (matrix memory): per token k, q [dim] and the two log gates;
// MODE 2 (decayed outer products): per token k, q [dim] and one decay.
// Shared memory, two stages of kRecTB tokens: per token [NV * DP key-side values (zero beyond dim) | 4 scalars], then v [kRecTB][CB].  The
// next stage arrives by cp.async while the current one is consumed.
constexpr int kRecTB = 16;

__device__ __forceinline__ void cp_async4_r(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async16_r(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_r() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_r() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DP, int LANES, int CPT, int MODE>
__global__ void __launch_bounds__(256)
column_recurrence_kernel(const float *__restrict__ rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off,
                         float *__restrict__ S, float *__restrict__ n_state, float *__restrict__ m_state, float *__restrict__ o,
                         float *__restrict__ nq_out, float *__restrict__ m_out, const int *__restrict__ seq_start,
                         const int *__restrict__ seq_pos0, const int *__restrict__ seq_slot, int heads, int kv_heads, int dim, int vdim) {
    constexpr int RPT = DP / LANES, NV = MODE == 0 ? 3 : 2, TS = NV * DP + 4;
    static_assert(RPT >= 4 && RPT % 4 == 0 && RPT * CPT <= 128, "state tile per thread");
    extern __shared__ __align__(16) float stage[];  // [2][kRecTB][TS] | v [2][kRecTB][CB]
    const int CB = blockDim.x / LANES * CPT;  // columns of this CTA
    float *vs = stage + 2 * kRecTB * TS;
    const int s = blockIdx.z, h = blockIdx.y, g = h / (heads / kv_heads);
    const int t0 = seq_start[s], len = seq_start[s + 1] - t0;
    if (len <= 0) return;
    const int pos0 = seq_pos0[s], slot = seq_slot[s];
    const int ncols = MODE == 1 ? vdim + 1 : vdim;
    const int cl = threadIdx.x / LANES * CPT, sub = threadIdx.x % LANES;  // first column within the CTA, lane within the column group
    const int col = blockIdx.x * CB + cl;
    auto row_of = [&](int i) { return 4 * (sub + LANES * (i >> 2)) + (i & 3); };  // the row that register row i of this lane holds
    float *Sp = S + ((size_t)slot * heads + h) * dim * vdim;
    float *np = MODE == 1 ? n_state + ((size_t)slot * heads + h) * dim : nullptr;
    // 16-byte copies when every source segment starts on a 16-byte boundary (the row's segments do; a head's part of one does if dim % 4 == 0)
    const bool v16 = dim % 4 == 0 && rec_ld % 4 == 0 && ((q_off | k_off | a_off) & 3) == 0 && (reinterpret_cast<size_t>(rec) & 15) == 0;

    if (dim < DP) {  // the rows beyond dim are zeroed once and never copied over
        const int pad = DP - dim;
        for (int i = threadIdx.x; i < 2 * kRecTB * NV * pad; i += blockDim.x) {
            const int tt = i / (NV * pad), w = i - tt * (NV * pad), which = w / pad;
            stage[tt * TS + which * DP + dim + (w - which * pad)] = 0.0f;
        }
        __syncthreads();
    }
    // a thread copies the same piece of every token of a stage: the split of its index into (vector, row) is done once per stage
    auto fetch = [&](int c0, int buf) {  // tokens c0 .. c0 + kRecTB - 1 of the portion into stage `buf`
        const int nt = min(kRecTB, len - c0);
        float *dst = stage + buf * kRecTB * TS;
        const float *row0 = rec + (size_t)(t0 + c0) * rec_ld;
        const int per = v16 ? dim / 4 : dim;
        for (int j = threadIdx.x; j < NV * per; j += blockDim.x) {
            const int which = j / per, r = (j - which * per) * (v16 ? 4 : 1);
            const float *src = row0 + (which == 0 ? k_off + g * dim : (which == 1 ? q_off + g * dim : a_off + h * dim)) + r;
            float *d = dst + which * DP + r;
            if (v16) {
                for (int tt = 0; tt < nt; ++tt) cp_async16_r(d + tt * TS, src + (size_t)tt * rec_ld);
            } else {
                for (int tt = 0; tt < nt; ++tt) cp_async4_r(d + tt * TS, src + (size_t)tt * rec_ld);
            }
        }
        if (threadIdx.x < 2) {
            const int w = threadIdx.x;
            const float *src = row0 + (MODE == 0 ? b_off + h : (w == 0 ? a_off + h : b_off + h));
            for (int tt = 0; tt < nt; ++tt) cp_async4_r(dst + tt * TS + NV * DP + w, src + (size_t)tt * rec_ld);
        }
        for (int cc = threadIdx.x; cc < CB; cc += blockDim.x) {
            const int c = blockIdx.x * CB + cc;
            for (int tt = 0; tt < nt; ++tt) {
                if (c < vdim) cp_async4_r(vs + (buf * kRecTB + tt) * CB + cc, row0 + (size_t)tt * rec_ld + v_off + h * vdim + c);
                else vs[(buf * kRecTB + tt) * CB + cc] = 1.0f;  // the normaliser's column: its value is 1
            }
        }
    };
    fetch(0, 0);
    cp_async_commit_r();

    // st[i][c]: row row_of(i), column col + c.  Column vdim of the matrix memory is the normaliser n
    float st[RPT][CPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = row_of(i);
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int cc = col + c;
            st[i][c] = (pos0 > 0 && cc < ncols && r < dim) ? ((MODE == 1 && cc == vdim) ? np[r] : Sp[(size_t)r * vdim + cc]) : 0.0f;
        }
    }
    float m = (MODE == 1 && pos0 > 0) ? m_state[(size_t)slot * heads + h] : 0.0f;

    for (int c0 = 0, buf = 0; c0 < len; c0 += kRecTB, buf ^= 1) {
        const int nt = min(kRecTB, len - c0);
        if (c0 + kRecTB < len) fetch(c0 + kRecTB, buf ^ 1);
        cp_async_commit_r();
        cp_async_wait_r<1>();
        __syncthreads();
        const float *sb = stage + buf * kRecTB * TS;
        // A token's staged vectors are read into registers one token ahead of their use: with one warp per scheduler nothing else hides
        // the shared-memory latency.  Piece j of a lane: float4 number sub + LANES * j of the staged vector.
        constexpr int NP = RPT / 4;
        auto load_token = [&](int tt, float4 *kk, float4 *qq, float4 *gg, float *vv, float &s0, float &s1) {
            const float4 *kp = reinterpret_cast<const float4 *>(sb + tt * TS) + sub;
#pragma unroll
            for (int j = 0; j < NP; ++j) {
                kk[j] = kp[LANES * j], qq[j] = kp[DP / 4 + LANES * j];
                if (MODE == 0) gg[j] = kp[2 * (DP / 4) + LANES * j];
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) vv[c] = vs[(buf * kRecTB + tt) * CB + cl + c];
            s0 = sb[tt * TS + NV * DP], s1 = sb[tt * TS + NV * DP + 1];
        };
        // (measured: reading ahead takes 30 % off a prompt of the decayed-memory mode with 8 lanes or fewer; with 16 lanes, where a lane holds
        // two pieces and the butterfly is longer, it adds 18 %, and it adds 6 % to the two longer token bodies)
        // (a lane that holds 64 rows has no registers left for a second set of pieces: it would spill)
        constexpr bool AHEAD = MODE == 2 && LANES <= 8 && RPT <= 32;
        float4 kc[NP], qc[NP], gc[NP];
        float v[CPT], s0c = 0.0f, s1c = 0.0f;
        if (AHEAD) load_token(0, kc, qc, gc, v, s0c, s1c);
#pragma unroll 4
        for (int tt = 0; tt < nt; ++tt) {  // unrolled: a token's read-out reduction overlaps the next token's first pass
            float4 kn[NP], qn[NP], gn[NP];
            float vn[CPT], s0n = 0.0f, s1n = 0.0f;
            const float4 *kp = reinterpret_cast<const float4 *>(sb + tt * TS) + sub, *qp = kp + DP / 4, *gp = kp + 2 * (DP / 4);
            if (AHEAD) {
                load_token(min(tt + 1, nt - 1), kn, qn, gn, vn, s0n, s1n);  // (the last token of a stage reads itself again)
            } else {  // the longer token bodies read their pieces where they use them
#pragma unroll
                for (int c = 0; c < CPT; ++c) v[c] = vs[(buf * kRecTB + tt) * CB + cl + c];
                s0c = sb[tt * TS + NV * DP], s1c = sb[tt * TS + NV * DP + 1];
            }
            float out[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) out[c] = 0.0f;
            if (MODE == 0) {
                const float beta = s0c;
                // four partial sums per dot product (one per row of a 16-byte piece): the chain of dependent multiply-adds is a quarter as long
                float dot4[4][CPT], out4[4][CPT];
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) dot4[e][c] = out4[e][c] = 0.0f;
                float dot[CPT];
                float kr[RPT];  // the key stays in registers for the second pass
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 kk = kp[LANES * (i >> 2)], gg = gp[LANES * (i >> 2)];
                    kr[i] = kk.x, kr[i + 1] = kk.y, kr[i + 2] = kk.z, kr[i + 3] = kk.w;
                    const float gv[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
#pragma unroll
                        for (int c = 0; c < CPT; ++c) {
                            st[i + e][c] *= gv[e];
                            dot4[e][c] = fmaf(kr[i + e], st[i + e][c], dot4[e][c]);
                        }
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c) dot[c] = (dot4[0][c] + dot4[1][c]) + (dot4[2][c] + dot4[3][c]);
#pragma unroll
                for (int w = LANES >> 1; w > 0; w >>= 1)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) dot[c] += __shfl_xor_sync(0xffffffffu, dot[c], w);
                float u[CPT];
#pragma unroll
                for (int c = 0; c < CPT; ++c) u[c] = beta * (v[c] - dot[c]);
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 qq = qp[LANES * (i >> 2)];
                    const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
#pragma unroll
                        for (int c = 0; c < CPT; ++c) {
                            st[i + e][c] = fmaf(kr[i + e], u[c], st[i + e][c]);
                            out4[e][c] = fmaf(qv[e], st[i + e][c], out4[e][c]);
                        }
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c) out[c] = (out4[0][c] + out4[1][c]) + (out4[2][c] + out4[3][c]);
            } else {
                float a, b;
                if (MODE == 1) {
                    const float gi = s0c, gf = s1c;
                    const float m_new = fmaxf(gf + m, gi);
                    a = expf(gf + m - m_new), b = expf(gi - m_new);
                    m = m_new;
                } else {
                    a = s0c, b = 1.0f;
                }
                float bv[CPT], out4[4][CPT];
#pragma unroll
                for (int c = 0; c < CPT; ++c) bv[c] = b * v[c];
#pragma unroll
                for (int e = 0; e < 4; ++e)
#pragma unroll
                    for (int c = 0; c < CPT; ++c) out4[e][c] = 0.0f;
#pragma unroll
                for (int i = 0; i < RPT; i += 4) {
                    const float4 kk = AHEAD ? kc[i >> 2] : kp[LANES * (i >> 2)], qq = AHEAD ? qc[i >> 2] : qp[LANES * (i >> 2)];
                    const float kv[4] = {kk.x, kk.y, kk.z, kk.w}, qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e)
#pragma unroll
                        for (int c = 0; c < CPT; ++c) {
                            st[i + e][c] = fmaf(a, st[i + e][c], kv[e] * bv[c]);
                            out4[e][c] = fmaf(qv[e], st[i + e][c], out4[e][c]);
                        }
                }
#pragma unroll
                for (int c = 0; c < CPT; ++c) out[c] = (out4[0][c] + out4[1][c]) + (out4[2][c] + out4[3][c]);
            }
#pragma unroll
            for (int w = LANES >> 1; w > 0; w >>= 1)
#pragma unroll
                for (int c = 0; c < CPT; ++c) out[c] += __shfl_xor_sync(0xffffffffu, out[c], w);
            if (sub == 0) {
                const size_t tok = (size_t)(t0 + c0 + tt);
#pragma unroll
                for (int c = 0; c < CPT; ++c) {
                    const int cc = col + c;
                    if (MODE == 1 && cc == vdim) nq_out[tok * heads + h] = out[c], m_out[tok * heads + h] = m;
                    else if (cc < vdim) o[(tok * heads + h) * vdim + cc] = out[c];
                }
            }
            if (AHEAD) {
#pragma unroll
                for (int j = 0; j < NP; ++j) kc[j] = kn[j], qc[j] = qn[j];
#pragma unroll
                for (int c = 0; c < CPT; ++c) v[c] = vn[c];
                s0c = s0n, s1c = s1n;
            }
        }
        __syncthreads();  // the stage is consumed: the fetch after next may overwrite it
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        const int r = row_of(i);
        if (r >= dim) continue;
#pragma unroll
        for (int c = 0; c < CPT; ++c) {
            const int cc = col + c;
            if (MODE == 1 && cc == vdim) np[r] = st[i][c];
            else if (cc < vdim) Sp[(size_t)r * vdim + cc] = st[i][c];
        }
    }
    if (MODE == 1 && sub == 0 && col <= vdim && vdim < col + CPT) m_state[(size_t)slot * heads + h] = m;
}

// One warp per (token, head): out[t, h*vdim + j] = out_scale * y_j * rsqrt(mean_j y^2 + eps) * w[h * w_stride + j] * sigmoid(gate) (gate_act 1: silu),
// y = o (delta) or o / (max(|nq|, exp(-m)) + 1e-6) (matrix memory: nq != NULL).  gate: fp32 pre-activations (gate_f) or the projection's.
template <typename T>
__global__ void __launch_bounds__(256)
head_output_kernel(const float *__restrict__ o, const float *__restrict__ nq, const float *__restrict__ m_in, const float *__restrict__ w,
                   int w_stride, float eps, const float *__restrict__ gate_f, int gate_f_ld, const T *__restrict__ gate_t, int gate_t_ld,
                   T *__restrict__ out, int out_ld, float out_scale, int tokens, int heads, int vdim, int gate_act) {
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
        out[(size_t)t * out_ld + h * vdim + j] = Elem<T>::from_f(src[j] * inv * w[h * w_stride + j] * (gate_act ? z * sigmoid_r(z) : sigmoid_r(z)) * out_scale);
    }
}

template <int DP, int LANES, int CPT, int MODE>
static int launch_colrec_t(const float *rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off, float *S, float *n_state,
                           float *m_state, float *o, float *nq, float *m_out, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                           int n_seqs, int heads, int kv_heads, int dim, int vdim, int one_token, cudaStream_t st) {
    const int ncols = MODE == 1 ? vdim + 1 : vdim, groups = (ncols + CPT - 1) / CPT;
    // every CTA stages its head's key-side vectors for itself, so CTAs are as wide as the batch allows while about a hundred of them remain
    const long long threads = (long long)groups * LANES * heads * n_seqs;
    int block = 256;
    while (block > 32 && block > LANES && threads / block < 100) block >>= 1;
    // a batch of one-token portions stages next to nothing: small CTAs leave fewer idle threads behind the last column (the normaliser's
    // column makes the column count odd) and fill the SMs evenly
    if (one_token && block > 64) block = 64;
    if (block < LANES) block = LANES;
    const int cb = block / LANES * CPT;
    constexpr int NV = MODE == 0 ? 3 : 2;
    const size_t smem = ((size_t)2 * kRecTB * (NV * DP + 4) + (size_t)2 * kRecTB * cb) * sizeof(float);
    auto kern = column_recurrence_kernel<DP, LANES, CPT, MODE>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<dim3((ncols + cb - 1) / cb, heads, n_seqs), block, smem, st>>>(rec, rec_ld, q_off, k_off, v_off, a_off, b_off, S, n_state, m_state, o, nq, m_out,
                                                                        seq_start, seq_pos0, seq_slot, heads, kv_heads, dim, vdim);
    return cuda_status("column_recurrence launch");
}

// how many lanes share a column group: at least what keeps a thread's state tile within its registers (rows per lane <= max_rows), then as
// many as it takes to give the device about two warps per SM, down to four rows per lane (one 16-byte piece of a staged vector)
static int pick_lanes(int dp, int max_rows, long long groups) {
    int lanes = dp > max_rows ? dp / max_rows : 1;
    if (const char *e = getenv("B200_RECURRENCE_LANES")) {  // measurement aid: a fixed lane count (a power of two within the limits)
        const int want = atoi(e);
        if (want >= lanes && want <= 32 && (want & (want - 1)) == 0 && dp / want >= 4) return want;
    }
    while (lanes < 16 && dp / (2 * lanes) >= 4 && groups * lanes < 148LL * 2 * 32) lanes *= 2;
    return lanes;
}

template <int MODE>
static int launch_colrec(const float *rec, int rec_ld, int q_off, int k_off, int v_off, int a_off, int b_off, float *S, float *n_state,
                         float *m_state, float *o, float *nq, float *m_out, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                         int n_seqs, int heads, int kv_heads, int dim, int vdim, int one_token, cudaStream_t st) {
    if (n_seqs == 0) return B200_OK;
    if (dim > 512) {
        set_error("column recurrence: key size %d above 512", dim);
        return B200_ERR_UNSUPPORTED;
    }
    const int dp = dim <= 16 ? 16 : (dim <= 32 ? 32 : (dim <= 64 ? 64 : (dim <= 128 ? 128 : (dim <= 256 ? 256 : 512))));
    const int ncols = vdim + (MODE == 1 ? 1 : 0);
    // one column per thread: measured against tiles of four columns (fewer shared-memory reads per multiply-add, but a quarter of the threads),
    // the single column won at every batch shape but one: the token loop is bound by its chain of dependent steps, not by its loads
    constexpr int cpt = 1;
    const int lanes = pick_lanes(dp, 64, (long long)n_seqs * heads * ncols);
#define B200_COLREC(D, L, C)  \
    if (dp == D && lanes == L && cpt == C) \
        return launch_colrec_t<D, L, C, MODE>(rec, rec_ld, q_off, k_off, v_off, a_off, b_off, S, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot, n_seqs, heads, kv_heads, dim, vdim, one_token, st)
    B200_COLREC(16, 1, 1); B200_COLREC(16, 2, 1); B200_COLREC(16, 4, 1);
    B200_COLREC(32, 1, 1); B200_COLREC(32, 2, 1); B200_COLREC(32, 4, 1); B200_COLREC(32, 8, 1);
    B200_COLREC(64, 1, 1); B200_COLREC(64, 2, 1); B200_COLREC(64, 4, 1); B200_COLREC(64, 8, 1); B200_COLREC(64, 16, 1);
    B200_COLREC(128, 2, 1); B200_COLREC(128, 4, 1); B200_COLREC(128, 8, 1); B200_COLREC(128, 16, 1); B200_COLREC(128, 32, 1);
    B200_COLREC(256, 4, 1); B200_COLREC(256, 8, 1); B200_COLREC(256, 16, 1); B200_COLREC(256, 32, 1);
    B200_COLREC(512, 8, 1); B200_COLREC(512, 16, 1); B200_COLREC(512, 32, 1);
#undef B200_COLREC
    set_error("column recurrence: no kernel for key size %d with %d lanes", dim, lanes);
    return B200_ERR_UNSUPPORTED;
}

int launch_delta_prep(int dtype, const void *proj, int ld, int col0, const float *conv_w, int taps, float *conv_state, const void *w_decay,
                      const float *decay_bias, const float *a_log, int rank, const void *w_gate2, int gate_rank, void *lr, float *za, float *zg,
                      float *rec, const int *tok_seq, const int *tok_pos, const int *seq_pos0, const int *seq_slot, int tokens, int heads,
                      int kv_heads, int dim, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const DeltaRow lay = delta_row(heads, kv_heads, dim, vdim);
    const size_t smem = ((size_t)2 * kv_heads * dim + heads * vdim) * sizeof(float), es = dtype == B200_F32 ? 4 : 2;
    void *lr_a = lr, *lr_g = (char *)lr + (((size_t)tokens * rank * es + 255) & ~(size_t)255);
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        // few tokens: few CTAs, so each gets more threads (a thread's channels are a chain of load latencies)
        delta_prep_kernel<T><<<tokens, tokens <= 64 ? 1024 : 256, smem, st>>>((const T *)proj, ld, col0, conv_w, taps, conv_state, rank, gate_rank, (T *)lr_a, (T *)lr_g, rec, lay,
                                                       tok_seq, tok_pos, seq_pos0, seq_slot, heads, kv_heads, dim, vdim);
    });
    int rc = cuda_status("delta_prep launch");
    if (rc != B200_OK) return rc;
    // the second halves of the two low-rank projections, fp32 out: tensor cores for 16-bit engines, the fp32 kernel otherwise
    const void *ws[2] = {w_decay, w_gate2}, *xs[2] = {lr_a, lr_g};
    float *zs[2] = {za, zg};
    const int ns[2] = {heads * dim, heads * vdim}, ks[2] = {rank, gate_rank};
    for (int i = 0; i < 2; ++i) {
        // (few tokens are a single 64-row tile on the tensor-core kernel -- few CTAs, each walking all of K: they take the fp32 kernel too)
        rc = tokens >= 64 ? launch_dense_f32out(dtype, xs[i], ws[i], zs[i], tokens, ns[i], ks[i], st) : B200_ERR_UNSUPPORTED;
        if (rc == B200_ERR_UNSUPPORTED) rc = launch_proj_f32(dtype, xs[i], ks[i], dtype, ws[i], nullptr, zs[i], ns[i], tokens, ns[i], ks[i], st);
        if (rc != B200_OK) return rc;
    }
    delta_finish_kernel<<<tokens, 256, 0, st>>>(za, zg, decay_bias, a_log, rec, lay, heads, dim, vdim);
    return cuda_status("delta_finish launch");
}

int launch_conv_state_update(int dtype, const void *proj, int ld, int col0, float *conv_state, int taps, int channels, const int *seq_start,
                             const int *seq_pos0, const int *seq_slot, int n_seqs, cudaStream_t st) {
    if (n_seqs == 0 || taps <= 1) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        conv_state_update_kernel<T><<<dim3((channels + 255) / 256, n_seqs), 256, 0, st>>>((const T *)proj, ld, col0, conv_state, taps, channels, seq_start, seq_pos0, seq_slot);
    });
    return cuda_status("conv_state_update launch");
}

int launch_delta_recurrent(const float *rec, float *S, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs,
                           int heads, int kv_heads, int dim, int vdim, cudaStream_t st, int one_token) {
    const DeltaRow lay = delta_row(heads, kv_heads, dim, vdim);
    return launch_colrec<0>(rec, lay.ld, lay.q, lay.k, lay.v, lay.decay, lay.beta, S, nullptr, nullptr, o, nullptr, nullptr, seq_start, seq_pos0,
                            seq_slot, n_seqs, heads, kv_heads, dim, vdim, one_token, st);
}

int launch_mlstm_prep(int dtype, const void *proj, int ld, int col0, const float *b_in, float cap, float *rec, int tokens, int heads, int dim,
                      int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const MlstmRow lay = mlstm_row(heads, dim, vdim);
    B200_DISPATCH_DTYPE(dtype, { mlstm_prep_kernel<T><<<tokens, 256, 0, st>>>((const T *)proj, ld, col0, b_in, cap, rec, lay, heads, dim, vdim); });
    return cuda_status("mlstm_prep launch");
}

int launch_mlstm_recurrent(const float *rec, float *S, float *n_state, float *m_state, float *o, float *nq, float *m_out, const int *seq_start,
                           const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim, cudaStream_t st, int one_token) {
    const MlstmRow lay = mlstm_row(heads, dim, vdim);
    return launch_colrec<1>(rec, lay.ld, lay.q, lay.k, lay.v, lay.gi, lay.gf, S, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot,
                            n_seqs, heads, heads, dim, vdim, one_token, st);
}

int launch_head_output(int dtype, const float *o, const float *nq, const float *m_in, const float *w, int w_stride, float eps,
                       const float *gate_f, int gate_f_ld, const void *gate_t, int gate_t_ld, void *out, int out_ld, float out_scale, int tokens,
                       int heads, int vdim, cudaStream_t st, int gate_act) {
    if (tokens == 0) return B200_OK;
    const int grid = (tokens * heads + 7) / 8;
    B200_DISPATCH_DTYPE(dtype, {
        head_output_kernel<T><<<grid, 256, 0, st>>>(o, nq, m_in, w, w_stride, eps, gate_f, gate_f_ld, (const T *)gate_t, gate_t_ld, (T *)out, out_ld,
                                                   out_scale, tokens, heads, vdim, gate_act);
    });
    return cuda_status("head_output launch");
}

int launch_delta_prep_direct(int dtype, const void *proj, int ld, int col0, const float *conv_w, int taps, float *conv_state,
                             const float *decay_bias, const float *a_log, float *rec, const int *tok_seq, const int *tok_pos,
                             const int *seq_pos0, const int *seq_slot, int tokens, int heads, int kv_heads, int dim, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const DeltaRow lay = delta_row(heads, kv_heads, dim, vdim);
    const size_t smem = ((size_t)2 * kv_heads * dim + heads * vdim) * sizeof(float);
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(delta_prep_direct_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        delta_prep_direct_kernel<T><<<tokens, tokens <= 64 ? 1024 : 256, smem, st>>>((const T *)proj, ld, col0, conv_w, taps, conv_state, decay_bias, a_log, rec,
                                                                                   lay, tok_seq, tok_pos, seq_pos0, seq_slot, heads, kv_heads, dim, vdim);
    });
    return cuda_status("delta_prep_direct launch");
}

int launch_ssd_prep(int dtype, const void *proj, int ld, int col0, const float *conv_w, const float *conv_b, int taps, float *conv_state,
                    const float *dt_bias, const float *a_log, const float *skip_w, float *rec, const int *tok_seq, const int *tok_pos,
                    const int *seq_pos0, const int *seq_slot, int tokens, int heads, int groups, int state, int vdim, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const DecayRow lay = decay_row(heads, groups, state, vdim);
    B200_DISPATCH_DTYPE(dtype, {
        ssd_prep_kernel<T><<<tokens, tokens <= 64 ? 1024 : 256, (size_t)heads * sizeof(float), st>>>((const T *)proj, ld, col0, conv_w, conv_b, taps, conv_state, dt_bias,
                                                                                                   a_log, skip_w, rec, lay, tok_seq, tok_pos, seq_pos0, seq_slot,
                                                                                                   heads, groups, state, vdim);
    });
    return cuda_status("ssd_prep launch");
}

int launch_linear_prep(int dtype, const void *proj, int ld, int col0, const float *head_decay, float *rec, int tokens, int heads, int dim, int vdim,
                       cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const DecayRow lay = decay_row(heads, heads, dim, vdim);
    B200_DISPATCH_DTYPE(dtype, { linear_prep_kernel<T><<<tokens, 256, 0, st>>>((const T *)proj, ld, col0, head_decay, rec, lay, heads, dim, vdim); });
    return cuda_status("linear_prep launch");
}

int launch_decay_recurrent(const float *rec, float *S, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs,
                           int heads, int kv_heads, int dim, int vdim, cudaStream_t st, int one_token) {
    const DecayRow lay = decay_row(heads, kv_heads, dim, vdim);
    return launch_colrec<2>(rec, lay.ld, lay.q, lay.k, lay.v, lay.decay, lay.decay, S, nullptr, nullptr, o, nullptr, nullptr, seq_start, seq_pos0,
                            seq_slot, n_seqs, heads, kv_heads, dim, vdim, one_token, st);
}

int launch_group_output(int dtype, const float *o, const float *skip, int skip_ld, const float *w, float eps, const void *gate, int gate_ld,
                        int gate_act, int gate_first, void *out, int out_ld, int tokens, int cols, int groups, cudaStream_t st) {
    if (tokens == 0) return B200_OK;
    const int per = cols / groups;
    // four columns per access when every piece of every row starts on a boundary of its access
    const bool vec = per % 4 == 0 && cols % 4 == 0 && skip_ld % 4 == 0 && gate_ld % 4 == 0 && out_ld % 4 == 0 && aligned16(o) && aligned16(skip) && aligned16(w) &&
                     ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(out)) & (dtype == B200_F32 ? 15 : 7)) == 0;
    const int pieces = vec ? per / 4 : per, threads = pieces <= 64 ? 32 : (pieces <= 128 ? 64 : (pieces <= 256 ? 128 : 256));
    B200_DISPATCH_DTYPE(dtype, {
        auto kern = vec ? group_output_kernel<T, true> : group_output_kernel<T, false>;
        kern<<<tokens * groups, threads, 0, st>>>(o, skip, skip_ld, w, eps, (const T *)gate, gate_ld, gate_act, gate_first, (T *)out, out_ld, cols, groups);
    });
    return cuda_status("group_output launch");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_delta_rule_recurrent(const float *rec, float *state, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                              int n_seqs, int heads, int kv_heads, int dim, int vdim, b200_stream_t stream) {
    B200_REQUIRE(rec && state && o && seq_start && seq_pos0 && seq_slot, "delta_rule_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "delta_rule_recurrent: bad shape");
    return launch_delta_recurrent(rec, state, o, seq_start, seq_pos0, seq_slot, n_seqs, heads, kv_heads, dim, vdim, as_stream(stream), 0);
}

int b200_decay_recurrent(const float *rec, float *state, float *o, const int *seq_start, const int *seq_pos0, const int *seq_slot,
                         int n_seqs, int heads, int kv_heads, int dim, int vdim, b200_stream_t stream) {
    B200_REQUIRE(rec && state && o && seq_start && seq_pos0 && seq_slot, "decay_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0, "decay_recurrent: bad shape");
    return launch_decay_recurrent(rec, state, o, seq_start, seq_pos0, seq_slot, n_seqs, heads, kv_heads, dim, vdim, as_stream(stream), 0);
}

int b200_mlstm_recurrent(const float *rec, float *state, float *n_state, float *m_state, float *o, float *nq, float *m_out,
                         const int *seq_start, const int *seq_pos0, const int *seq_slot, int n_seqs, int heads, int dim, int vdim,
                         b200_stream_t stream) {
    B200_REQUIRE(rec && state && n_state && m_state && o && nq && m_out && seq_start && seq_pos0 && seq_slot, "mlstm_recurrent: null pointer");
    B200_REQUIRE(n_seqs >= 0 && heads > 0 && dim > 0 && vdim > 0, "mlstm_recurrent: bad shape");
    return launch_mlstm_recurrent(rec, state, n_state, m_state, o, nq, m_out, seq_start, seq_pos0, seq_slot, n_seqs, heads, dim, vdim,
                                  as_stream(stream), 0);
}
}
