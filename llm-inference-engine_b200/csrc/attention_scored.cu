// attention_scored.cu -- grouped-query attention over a paged pool of keys [dim] and values [vdim] whose parts are options of the launch
// (B200_MIXER_ATTN_SCORED), for ragged mixed batches:
//   * scored_prep_kernel: bias of the q / k / v projections, RMS norm of every q and k head (one weight vector shared by the heads),
//     rotation of the first rot_dims dimensions of every q and k head in INTERLEAVED pairs (2i, 2i+1) -- or in halves (i, i + rot_dims/2) --
//     by the angle pos * base^(-2i/rot_dims), optionally with the long wavelengths slowed down; optionally every value head divided by its
//     root mean square; q to a dense buffer, k and v to their pages;
//   * scored_attn_kernel: every token of the batch against the keys of ITS sequence inside the window 0 <= i - j < window (0: all j <= i).
//     score = cap(scale * q.k) - r1[h] * ln(1 + r2[h] * (i - j)) (cap(s) = c tanh(s / c) and the penalty are optional); weights either softmax over the visible keys or
//     sigmoid(score + head_bias[h]) without any normalisation; optional sigmoid output gate; the result is scaled by out_scale and written
//     with a row stride, so that several mixers fill one row of a shared output-projection input;
//   * scored_attn_mma_kernel: the same for prompt portions on the tensor cores (16-bit engines, dim and vdim multiples of 16 up to 128).
// A token is (sequence, position): its keys are looked up through the sequence's block-table row and the rows a call appends are in the
// pool before any score is formed, so prompt portions and single decoded tokens are one case.
// Angles are formed in fp64 (a position times a frequency loses digits in fp32 at long contexts); norms, scores, weights and the weighted
// sum are fp32; q, k, v and the output are of the engine dtype.
#include "hybrid_ops.cuh"

#include <algorithm>

namespace b200 {

constexpr int kPageS = B200_KV_PAGE_SIZE;

template <typename T>
__global__ void __launch_bounds__(256)
scored_prep_kernel(const T *__restrict__ proj, int ld, int col0, const float *__restrict__ b_in, T *__restrict__ q_out, T *__restrict__ k_pool,
                   T *__restrict__ v_pool, const float *__restrict__ q_norm, const float *__restrict__ k_norm, float eps,
                   const int *__restrict__ tok_seq, const int *__restrict__ tok_pos, const int *__restrict__ block_table, int mpps, int heads,
                   int kv_heads, int dim, int vdim, int rot_dims, float rot_base, ScoredPrepOptions opt) {
    extern __shared__ float rot[];  // cos [rot_dims/2] | sin [rot_dims/2]
    const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    const int pos = tok_pos[t], half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        double f = pow((double)rot_base, -2.0 * (double)i / (double)rot_dims);
        if (opt.rot_factor > 0.0f) {  // long wavelengths turn more slowly, with a smooth band between the two regimes
            const double wl = 6.283185307179586476925286766559 / f, orig = (double)opt.rot_original;
            if (wl > orig / (double)opt.rot_low) {
                f /= (double)opt.rot_factor;
            } else if (!(wl < orig / (double)opt.rot_high)) {
                const double sm = (orig / wl - (double)opt.rot_low) / ((double)opt.rot_high - (double)opt.rot_low);
                f = (1.0 - sm) * f / (double)opt.rot_factor + sm * f;
            }
        }
        const double a = (double)pos * f;
        double s, c;
        sincos(a, &s, &c);
        rot[i] = (float)c, rot[half + i] = (float)s;
    }
    __syncthreads();
    const T *row = proj + (size_t)t * ld + col0;
    const float *bias = b_in;  // counted from the mixer's own first row
    const int page = block_table[(size_t)tok_seq[t] * mpps + pos / kPageS], off = pos % kPageS;
    for (int hh = warp; hh < heads + kv_heads; hh += nwarp) {
        const bool is_q = hh < heads;
        const int src = is_q ? hh * dim : heads * dim + (hh - heads) * dim;
        const float *nw = is_q ? q_norm : k_norm;
        float inv = 1.0f;
        if (nw) {
            float ss = 0.0f;
            for (int c = lane; c < dim; c += 32) {
                const float v = Elem<T>::to_f(row[src + c]) + (bias ? bias[src + c] : 0.0f);
                ss = fmaf(v, v, ss);
            }
            inv = rsqrtf(warp_sum(ss) / (float)dim + eps);
        }
        T *dst;
        if (is_q) dst = q_out + ((size_t)t * heads + hh) * dim;
        else if (page >= 0) dst = k_pool + (((size_t)page * kv_heads + (hh - heads)) * kPageS + off) * dim;
        else continue;  // no page held: nothing is written (the host refuses such a batch)
        auto load = [&](int c) {
            const float v = Elem<T>::to_f(row[src + c]) + (bias ? bias[src + c] : 0.0f);
            return nw ? v * inv * nw[c] : v;
        };
        for (int p = lane; p < half; p += 32) {  // the rotating pairs: (2p, 2p+1), or (p, p + half)
            const int c0 = opt.rot_half ? p : 2 * p, c1 = opt.rot_half ? p + half : 2 * p + 1;
            const float a = load(c0), b = load(c1), cs = rot[p], sn = rot[half + p];
            dst[c0] = Elem<T>::from_f(a * cs - b * sn);
            dst[c1] = Elem<T>::from_f(b * cs + a * sn);
        }
        for (int c = rot_dims + lane; c < dim; c += 32) dst[c] = Elem<T>::from_f(load(c));  // the rest passes unchanged
    }
    if (page < 0) return;
    const int vsrc = (heads + kv_heads) * dim;
    if (opt.v_norm) {  // every value head is cached divided by its root mean square
        for (int g = warp; g < kv_heads; g += nwarp) {
            float ss = 0.0f;
            for (int c = lane; c < vdim; c += 32) {
                const float v = Elem<T>::to_f(row[vsrc + g * vdim + c]) + (bias ? bias[vsrc + g * vdim + c] : 0.0f);
                ss = fmaf(v, v, ss);
            }
            const float inv = rsqrtf(warp_sum(ss) / (float)vdim + eps);
            for (int c = lane; c < vdim; c += 32) {
                const float v = Elem<T>::to_f(row[vsrc + g * vdim + c]) + (bias ? bias[vsrc + g * vdim + c] : 0.0f);
                v_pool[(((size_t)page * kv_heads + g) * kPageS + off) * vdim + c] = Elem<T>::from_f(v * inv);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < kv_heads * vdim; c += blockDim.x) {
        const int g = c / vdim, cc = c - g * vdim;
        const float v = Elem<T>::to_f(row[vsrc + c]) + (bias ? bias[vsrc + c] : 0.0f);
        v_pool[(((size_t)page * kv_heads + g) * kPageS + off) * vdim + cc] = Elem<T>::from_f(v);
    }
}

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
// for weights that are rounded to 16 bits right away: hardware exponential and reciprocal (relative error ~1e-6)
__device__ __forceinline__ float sigmoid_fast(float z) { return __fdividef(1.0f, 1.0f + __expf(-z)); }
// tanh(z) = sign(z) (1 - 2 / (exp(2|z|) + 1)) from the hardware exponential and reciprocal: absolute error of a few 1e-7, saturating cleanly
__device__ __forceinline__ float tanh_fast(float z) {
    const float e = __expf(2.0f * fabsf(z));
    return copysignf(1.0f - __fdividef(2.0f, e + 1.0f), z);
}

// One CTA per (token, query head).  Shared memory: q[dim] | weights[keys] | partial[key groups][vdim] | red[33].
template <typename T>
__global__ void __launch_bounds__(512)
scored_attn_kernel(const T *__restrict__ q, const T *__restrict__ k_pool, const T *__restrict__ v_pool, const float *__restrict__ head_bias,
                   const float *__restrict__ dist_r1, const float *__restrict__ dist_r2, const T *__restrict__ gate_in, int gate_ld,
                   T *__restrict__ out, int out_ld, float out_scale, const int *__restrict__ tok_seq, const int *__restrict__ tok_pos,
                   const int *__restrict__ block_table, int mpps, int heads, int kv_heads, int dim, int vdim, float scale, int window,
                   int sigmoid, int max_keys, int part_floats, const int *__restrict__ tok_list, float softcap) {
    extern __shared__ float sm[];
    const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, h = blockIdx.y;
    const int g = h / (heads / kv_heads);
    const int pos = tok_pos[t];
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    const int nkeys = pos - first + 1;
    float *qs = sm;
    float *sc = qs + dim;
    float *part = sc + max_keys;
    float *red = part + part_floats;
    const int *bt = block_table + (size_t)tok_seq[t] * mpps;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) qs[c] = Elem<T>::to_f(q[((size_t)t * heads + h) * dim + c]);
    __syncthreads();
    const float r1 = dist_r1 ? dist_r1[h] : 0.0f, r2 = dist_r2 ? dist_r2[h] : 0.0f, hb = head_bias ? head_bias[h] : 0.0f;
    constexpr int V = Elem<T>::kVec;
    const bool kvec = dim % V == 0, vvec = vdim % V == 0;

    // ---- scores: four adjacent lanes share a key row
    float mx = -INFINITY;
    {
        const int sub = threadIdx.x & 3, kslot = threadIdx.x >> 2, nslots = blockDim.x >> 2, pieces = dim / V;
        for (int j0 = 0; j0 < nkeys; j0 += nslots) {  // warp-uniform trip count: the shuffles below take every lane
            const int j = j0 + kslot;
            const int p = first + min(j, nkeys - 1);
            const T *kr = k_pool + (((size_t)bt[p / kPageS] * kv_heads + g) * kPageS + (p % kPageS)) * dim;
            float a0 = 0.0f, a1 = 0.0f;
            if (kvec) {
#pragma unroll 4
                for (int pc = sub; pc < pieces; pc += 4) {
                    float f[V];
                    unpack16<T>(ld_v4(kr + pc * V), f);
                    const float *qp = qs + pc * V;
#pragma unroll
                    for (int i = 0; i < V; i += 2) a0 = fmaf(qp[i], f[i], a0), a1 = fmaf(qp[i + 1], f[i + 1], a1);
                }
            } else {
                for (int c = sub; c < dim; c += 4) a0 = fmaf(qs[c], Elem<T>::to_f(kr[c]), a0);
            }
            float acc = a0 + a1;
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc *= scale;
            if (softcap > 0.0f) acc = softcap * tanhf(acc / softcap);
            if (dist_r1) acc -= r1 * log1pf(r2 * (float)(pos - p));
            if (sigmoid) acc = sigmoid_f(acc + hb);
            if (j < nkeys) {
                if (sub == 0) sc[j] = acc;
                mx = fmaxf(mx, acc);
            }
        }
    }
    float inv = 1.0f;
    if (!sigmoid) {
        mx = block_max(mx, red);
        float sum = 0.0f;
        for (int j = threadIdx.x; j < nkeys; j += blockDim.x) {
            const float e = expf(sc[j] - mx);
            sc[j] = e;
            sum += e;
        }
        inv = 1.0f / block_sum(sum, red);  // (its barriers also publish sc[])
    } else {
        __syncthreads();
    }

    // ---- weighted sum of the values
    const int tpr = vdim / V;  // threads per value row when a thread takes one 16-byte piece
    if (vvec && tpr <= (int)blockDim.x) {
        const int groups = (int)blockDim.x / tpr, kg = threadIdx.x / tpr, c0 = (threadIdx.x - kg * tpr) * V;
        float acc[V];
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = 0.0f;
        if (kg < groups) {
#pragma unroll 8
            for (int j = kg; j < nkeys; j += groups) {
                const int p = first + j;
                float f[V];
                unpack16<T>(ld_v4(v_pool + (((size_t)bt[p / kPageS] * kv_heads + g) * kPageS + (p % kPageS)) * vdim + c0), f);
                const float w = sc[j];
#pragma unroll
                for (int i = 0; i < V; ++i) acc[i] = fmaf(w, f[i], acc[i]);
            }
#pragma unroll
            for (int i = 0; i < V; ++i) part[kg * vdim + c0 + i] = acc[i];
        }
        __syncthreads();
        for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
            float a = 0.0f;
            for (int k2 = 0; k2 < groups; ++k2) a += part[k2 * vdim + c];
            part[c] = a;  // column c's entries are read by this thread only
        }
        __syncthreads();
    } else {
        const int ngroups = (int)blockDim.x >= vdim ? (int)blockDim.x / vdim : 1;
        if (ngroups > 1) {
            const int kg = threadIdx.x / vdim, c = threadIdx.x - kg * vdim;
            if (kg < ngroups) {
                float acc = 0.0f;
                for (int j = kg; j < nkeys; j += ngroups) {
                    const int p = first + j;
                    acc = fmaf(sc[j], Elem<T>::to_f(v_pool[(((size_t)bt[p / kPageS] * kv_heads + g) * kPageS + (p % kPageS)) * vdim + c]), acc);
                }
                part[kg * vdim + c] = acc;
            }
            __syncthreads();
            if ((int)threadIdx.x < vdim) {
                float acc = 0.0f;
                for (int k2 = 0; k2 < ngroups; ++k2) acc += part[k2 * vdim + threadIdx.x];
                part[threadIdx.x] = acc;
            }
            __syncthreads();
        } else {
            for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
                float acc = 0.0f;
                for (int j = 0; j < nkeys; ++j) {
                    const int p = first + j;
                    acc = fmaf(sc[j], Elem<T>::to_f(v_pool[(((size_t)bt[p / kPageS] * kv_heads + g) * kPageS + (p % kPageS)) * vdim + c]), acc);
                }
                part[c] = acc;
            }
            __syncthreads();
        }
    }
    for (int c = threadIdx.x; c < vdim; c += blockDim.x) {
        float o = part[c] * inv;
        if (gate_in) o *= sigmoid_f(Elem<T>::to_f(gate_in[(size_t)t * gate_ld + h * vdim + c]));
        out[(size_t)t * out_ld + h * vdim + c] = Elem<T>::from_f(o * out_scale);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// Tensor-core kernel for prompt portions (16-bit engines): one CTA = 64 consecutive tokens of ONE sequence x one query head, four warps
// of 16 rows each.  A key tile is one page (64 positions): K and V arrive by cp.async into a two-stage ring, S = Q K^T and O += P V run on
// mma.sync.m16n8k16 with fp32 accumulators.  SOFTMAX: the online form in fp32 (base 2); the distance penalty of a head is a table over the
// distance in shared memory.  SIGMOID: P = sigmoid(score + head_bias) goes to the second product as it is: no running state at all.
// The mask is evaluated per element; the tiles walked are those from the window start of the tile's first query to its last query.
// tiles: int4 per tile {sequence, first packed row, rows (1..64), position of the first row}.
constexpr int kTileQS = 64;

__device__ __forceinline__ void cp_async16_s(void *smem, const void *gmem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit_s() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_s() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void ldsm4_trans(unsigned &r0, unsigned &r1, unsigned &r2, unsigned &r3, const void *p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
template <typename T> __device__ __forceinline__ void mma16816(float *c, const unsigned *a, unsigned b0, unsigned b1);
template <> __device__ __forceinline__ void mma16816<__nv_bfloat16>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void mma16816<__half>(float *c, const unsigned *a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ unsigned pack2s(float lo, float hi);
template <> __device__ __forceinline__ unsigned pack2s<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}
template <> __device__ __forceinline__ unsigned pack2s<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned *>(&v);
}
// element (row, col) of a [rows][D] 16-bit tile (D = 32, 64 or 128) whose 16-byte pieces are XOR-swizzled by the row inside groups of up to
// eight pieces
template <int D> __device__ __forceinline__ int swzs(int row, int col) {
    constexpr int M = D / 8 >= 8 ? 7 : D / 8 - 1;
    const int piece = col >> 3;
    return row * D + ((((piece & ~M) | ((piece ^ row) & M)) << 3) | (col & 7));
}

template <typename T, int DK, int DV, int SIG>
__global__ void __launch_bounds__(128)
scored_attn_mma_kernel(const T *__restrict__ q, const T *__restrict__ k_pool, const T *__restrict__ v_pool, const float *__restrict__ head_bias,
                       const float *__restrict__ dist_r1, const float *__restrict__ dist_r2, const T *__restrict__ gate_in, int gate_ld,
                       T *__restrict__ out, int out_ld, float out_scale, const int4 *__restrict__ tiles, const int *__restrict__ block_table,
                       int mpps, int heads, int kv_heads, float scale, int window, int pen_len, float softcap) {
    extern __shared__ __align__(16) unsigned char smraw[];
    T *qs = reinterpret_cast<T *>(smraw);       // [64][DK]
    T *ks = qs + kTileQS * DK;                  // [2][64][DK]
    T *vs = ks + 2 * kPageS * DK;               // [2][64][DV]
    float *pen = reinterpret_cast<float *>(vs + 2 * kPageS * DV);  // [pen_len]: the distance penalty in base-2 units
    const int4 tile = tiles[blockIdx.x];
    const int h = blockIdx.y, g = h / (heads / kv_heads);
    const int row0 = tile.y, nrows = tile.z, pos0 = tile.w;
    const int *bt = block_table + (size_t)tile.x * mpps;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    constexpr int kPK = DK / 8, kPV = DV / 8;
    constexpr float kLog2e = 1.4426950408889634f;

    const int last = pos0 + nrows - 1;
    const int first = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int tile_lo = first / kPageS, tile_hi = last / kPageS;

    auto load_kv = [&](int kt, int stage) {
        const int page = bt[kt];
        const T *kg = k_pool + ((size_t)page * kv_heads + g) * kPageS * DK;
        const T *vg = v_pool + ((size_t)page * kv_heads + g) * kPageS * DV;
        for (int i = threadIdx.x; i < kPageS * kPK; i += 128) {
            const int r = i / kPK, c = (i % kPK) * 8;
            // rows past the tile's last query have not been written (or belong to a page's previous owner); their weights are zero, but
            // 0 x NaN is NaN on the tensor core (and a sigmoid of garbage is not zero), so keys and values there are zeroed, not fetched
            if (kt * kPageS + r <= last) cp_async16_s(ks + stage * kPageS * DK + swzs<DK>(r, c), kg + r * DK + c);
            else *reinterpret_cast<uint4 *>(ks + stage * kPageS * DK + swzs<DK>(r, c)) = make_uint4(0, 0, 0, 0);
        }
        for (int i = threadIdx.x; i < kPageS * kPV; i += 128) {
            const int r = i / kPV, c = (i % kPV) * 8;
            if (kt * kPageS + r <= last) cp_async16_s(vs + stage * kPageS * DV + swzs<DV>(r, c), vg + r * DV + c);
            else *reinterpret_cast<uint4 *>(vs + stage * kPageS * DV + swzs<DV>(r, c)) = make_uint4(0, 0, 0, 0);
        }
    };
    load_kv(tile_lo, 0);
    cp_async_commit_s();
    for (int i = threadIdx.x; i < kTileQS * kPK; i += 128) {
        const int r = i / kPK, c = (i % kPK) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < nrows) v = ld_v4(q + ((size_t)(row0 + r) * heads + h) * DK + c);
        *reinterpret_cast<uint4 *>(qs + swzs<DK>(r, c)) = v;
    }
    if (!SIG && dist_r1) {
        const float r1 = dist_r1[h] * kLog2e, r2 = dist_r2[h];
        for (int d = threadIdx.x; d < pen_len; d += 128) pen[d] = r1 * log1pf(r2 * (float)d);
    }
    __syncthreads();
    unsigned qf[DK / 16][4];
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk)
        ldsm4(qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], qs + swzs<DK>(warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, kk * 16 + (lane >> 4) * 8));

    // a capped score: cap * tanh(scale * s / cap), in the softmax form times log2(e)
    const bool capped = softcap > 0.0f;
    const float sl2 = capped ? scale / softcap : (SIG ? scale : scale * kLog2e), cap2 = SIG ? softcap : softcap * kLog2e;
    auto scaled = [&](float sv) { return capped ? cap2 * tanh_fast(sv * sl2) : sv * sl2; };
    const float hb = (SIG && head_bias) ? head_bias[h] : 0.0f;
    const bool has_pen = !SIG && dist_r1 != nullptr;
    const int p_a = pos0 + warp * 16 + gid, p_b = p_a + 8;  // rows gid and gid + 8 of this warp's 16
    const int lo_a = window > 0 ? p_a - window + 1 : 0, lo_b = window > 0 ? p_b - window + 1 : 0;
    float m_a = -1e30f, m_b = -1e30f, l_a = 0.0f, l_b = 0.0f;
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    for (int kt = tile_lo; kt <= tile_hi; ++kt) {
        const int stage = (kt - tile_lo) & 1;
        if (kt < tile_hi) load_kv(kt + 1, stage ^ 1);
        cp_async_commit_s();
        cp_async_wait_s<1>();
        __syncthreads();
        const T *kst = ks + stage * kPageS * DK, *vst = vs + stage * kPageS * DV;
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {  // two key blocks of 8 per ldmatrix
                unsigned b0, b1, b2, b3;
                ldsm4(b0, b1, b2, b3, kst + swzs<DK>(jp * 16 + (lane & 7) + (lane >> 4) * 8, kk * 16 + ((lane >> 3) & 1) * 8));
                mma16816<T>(s[2 * jp], qf[kk], b0, b1);
                mma16816<T>(s[2 * jp + 1], qf[kk], b2, b3);
            }
        }
        unsigned pf[4][4];
        if (SIG) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float w[4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kt * kPageS + j * 8 + tig * 2 + e;
                    w[e] = (key <= p_a && key >= lo_a) ? sigmoid_fast(scaled(s[j][e]) + hb) : 0.0f;
                    w[2 + e] = (key <= p_b && key >= lo_b) ? sigmoid_fast(scaled(s[j][2 + e]) + hb) : 0.0f;
                }
                pf[j >> 1][(j & 1) * 2] = pack2s<T>(w[0], w[1]);
                pf[j >> 1][(j & 1) * 2 + 1] = pack2s<T>(w[2], w[3]);
            }
        } else {
            float mx_a = m_a, mx_b = m_b;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = kt * kPageS + j * 8 + tig * 2 + e;
                    const bool va = key <= p_a && key >= lo_a, vb = key <= p_b && key >= lo_b;
                    s[j][e] = va ? scaled(s[j][e]) - (has_pen ? pen[p_a - key] : 0.0f) : -INFINITY;
                    s[j][2 + e] = vb ? scaled(s[j][2 + e]) - (has_pen ? pen[p_b - key] : 0.0f) : -INFINITY;
                    mx_a = fmaxf(mx_a, s[j][e]);
                    mx_b = fmaxf(mx_b, s[j][2 + e]);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            const float f_a = exp2f(m_a - mx_a), f_b = exp2f(m_b - mx_b);
            m_a = mx_a, m_b = mx_b;
            float sum_a = 0.0f, sum_b = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float e0 = exp2f(s[j][0] - m_a), e1 = exp2f(s[j][1] - m_a), e2 = exp2f(s[j][2] - m_b), e3 = exp2f(s[j][3] - m_b);
                sum_a += e0 + e1, sum_b += e2 + e3;
                pf[j >> 1][(j & 1) * 2] = pack2s<T>(e0, e1);
                pf[j >> 1][(j & 1) * 2 + 1] = pack2s<T>(e2, e3);
            }
            l_a = l_a * f_a + sum_a, l_b = l_b * f_b + sum_b;  // per-lane partial sums; joined across the row's four lanes at the end
#pragma unroll
            for (int j = 0; j < DV / 8; ++j) o[j][0] *= f_a, o[j][1] *= f_a, o[j][2] *= f_b, o[j][3] *= f_b;
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {      // 16 keys per step
#pragma unroll
            for (int jp = 0; jp < DV / 16; ++jp) {
                unsigned b0, b1, b2, b3;
                ldsm4_trans(b0, b1, b2, b3, vst + swzs<DV>(kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, jp * 16 + (lane >> 4) * 8));
                mma16816<T>(o[2 * jp], pf[kk], b0, b1);
                mma16816<T>(o[2 * jp + 1], pf[kk], b2, b3);
            }
        }
        __syncthreads();  // everybody is done with this stage before the next iteration's prefetch overwrites it
    }
    float i_a = 1.0f, i_b = 1.0f;
    if (!SIG) {
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
        l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
        l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
        i_a = 1.0f / l_a, i_b = 1.0f / l_b;
    }
    i_a *= out_scale, i_b *= out_scale;
    const int r_a = warp * 16 + gid, r_b = r_a + 8;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j) {
        const int c = j * 8 + tig * 2;
        if (r_a < nrows) {
            float x0 = o[j][0] * i_a, x1 = o[j][1] * i_a;
            if (gate_in) {
                const T *gp = gate_in + (size_t)(row0 + r_a) * gate_ld + h * DV + c;
                x0 *= sigmoid_f(Elem<T>::to_f(gp[0])), x1 *= sigmoid_f(Elem<T>::to_f(gp[1]));
            }
            *reinterpret_cast<unsigned *>(out + (size_t)(row0 + r_a) * out_ld + h * DV + c) = pack2s<T>(x0, x1);
        }
        if (r_b < nrows) {
            float x2 = o[j][2] * i_b, x3 = o[j][3] * i_b;
            if (gate_in) {
                const T *gp = gate_in + (size_t)(row0 + r_b) * gate_ld + h * DV + c;
                x2 *= sigmoid_f(Elem<T>::to_f(gp[0])), x3 *= sigmoid_f(Elem<T>::to_f(gp[1]));
            }
            *reinterpret_cast<unsigned *>(out + (size_t)(row0 + r_b) * out_ld + h * DV + c) = pack2s<T>(x2, x3);
        }
    }
}

static bool tile_dim_ok(int d) { return d == 32 || d == 64 || d == 128; }

bool scored_attention_tiles_supported(int dtype, int dim, int vdim, int gate_ld, int out_ld, int window, bool penalty) {
    // the penalty table of a windowed layer lives in shared memory; without a window it would be as long as the context
    return dtype != B200_F32 && tile_dim_ok(dim) && tile_dim_ok(vdim) && gate_ld % 2 == 0 && out_ld % 2 == 0 &&
           (!penalty || (window > 0 && window <= 8192));
}

template <typename T, int DK, int DV>
static int launch_scored_mma_t(const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *r1, const float *r2,
                               const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale, const int *tiles, int n_tiles,
                               const int *block_table, int mpps, int heads, int kv_heads, float scale, int window, int sigmoid, cudaStream_t st,
                               float softcap) {
    const int pen_len = (!sigmoid && r1) ? window + kTileQS : 0;
    const size_t smem = (size_t)(kTileQS + 2 * kPageS) * DK * sizeof(T) + (size_t)2 * kPageS * DV * sizeof(T) + (size_t)pen_len * sizeof(float);
    auto kern = sigmoid ? scored_attn_mma_kernel<T, DK, DV, 1> : scored_attn_mma_kernel<T, DK, DV, 0>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kern<<<dim3(n_tiles, heads), 128, smem, st>>>((const T *)q, (const T *)k_pool, (const T *)v_pool, head_bias, r1, r2, (const T *)gate_in, gate_ld,
                                                  (T *)out, out_ld, out_scale, (const int4 *)tiles, block_table, mpps, heads, kv_heads, scale, window,
                                                  pen_len, softcap);
    return cuda_status("scored_attention (tensor core) launch");
}

int launch_scored_attention_tiles(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                                  const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale,
                                  const int *tiles, int n_tiles, const int *block_table, int mpps, int heads, int kv_heads, int dim, int vdim,
                                  float scale, int window, int sigmoid, cudaStream_t st, float softcap) {
    if (n_tiles == 0) return B200_OK;
    if (!scored_attention_tiles_supported(dtype, dim, vdim, gate_ld, out_ld, window, dist_r1 != nullptr)) {
        set_error("scored_attention tiles: 16-bit dtypes, dim and vdim of 32 / 64 / 128, a penalty only with a window");
        return B200_ERR_UNSUPPORTED;
    }
#define B200_SCORED_ARGS q, k_pool, v_pool, head_bias, dist_r1, dist_r2, gate_in, gate_ld, out, out_ld, out_scale, tiles, n_tiles, block_table, mpps, heads, kv_heads, scale, window, sigmoid, st, softcap
#define B200_SCORED_DV(TT, DK)                                                     \
    do {                                                                           \
        if (vdim == 32) return launch_scored_mma_t<TT, DK, 32>(B200_SCORED_ARGS);  \
        if (vdim == 64) return launch_scored_mma_t<TT, DK, 64>(B200_SCORED_ARGS);  \
        return launch_scored_mma_t<TT, DK, 128>(B200_SCORED_ARGS);                 \
    } while (0)
#define B200_SCORED_DK(TT)                      \
    do {                                        \
        if (dim == 32) B200_SCORED_DV(TT, 32);  \
        if (dim == 64) B200_SCORED_DV(TT, 64);  \
        B200_SCORED_DV(TT, 128);                \
    } while (0)
    if (dtype == B200_BF16) B200_SCORED_DK(__nv_bfloat16);
    B200_SCORED_DK(__half);
#undef B200_SCORED_DK
#undef B200_SCORED_DV
#undef B200_SCORED_ARGS
}

int launch_scored_prep(int dtype, const void *proj, int ld, int col0, const float *b_in, void *q_out, void *k_pool, void *v_pool,
                       const float *q_norm, const float *k_norm, float eps, const int *tok_seq, const int *tok_pos, const int *block_table,
                       int mpps, int tokens, int heads, int kv_heads, int dim, int vdim, int rot_dims, float rot_base, cudaStream_t st,
                       ScoredPrepOptions opt) {
    if (tokens == 0) return B200_OK;
    B200_DISPATCH_DTYPE(dtype, {
        scored_prep_kernel<T><<<tokens, 256, (size_t)std::max(rot_dims, 2) * sizeof(float), st>>>(
            (const T *)proj, ld, col0, b_in, (T *)q_out, (T *)k_pool, (T *)v_pool, q_norm, k_norm, eps, tok_seq, tok_pos, block_table, mpps, heads,
            kv_heads, dim, vdim, rot_dims, rot_base, opt);
    });
    return cuda_status("scored_prep launch");
}

int launch_scored_attention(int dtype, const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                            const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale, const int *tok_seq,
                            const int *tok_pos, const int *block_table, int mpps, int tokens, int heads, int kv_heads, int dim, int vdim,
                            float scale, int window, int sigmoid, int max_keys, cudaStream_t st, const int *tok_list, float softcap) {
    if (tokens == 0) return B200_OK;
    const int threads = max_keys >= 512 ? 512 : (max_keys >= 256 ? 256 : 128);  // long contexts: more keys in flight per CTA
    const int ngroups = threads >= vdim ? threads / vdim : 1;
    const size_t part = std::max((size_t)ngroups * vdim, (size_t)threads * 8);  // key-group partial sums (scalar / 16-byte path)
    const size_t smem = ((size_t)dim + max_keys + part + 33) * sizeof(float);
    if (smem > 200 * 1024) {
        set_error("scored_attention: %d keys x dim %d do not fit the shared-memory weight buffer", max_keys, dim);
        return B200_ERR_UNSUPPORTED;
    }
    B200_DISPATCH_DTYPE(dtype, {
        if (smem > 48 * 1024) cudaFuncSetAttribute(scored_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        scored_attn_kernel<T><<<dim3(tokens, heads), threads, smem, st>>>(
            (const T *)q, (const T *)k_pool, (const T *)v_pool, head_bias, dist_r1, dist_r2, (const T *)gate_in, gate_ld, (T *)out, out_ld, out_scale,
            tok_seq, tok_pos, block_table, mpps, heads, kv_heads, dim, vdim, scale, window, sigmoid, max_keys, (int)part, tok_list, softcap);
    });
    return cuda_status("scored_attention launch");
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_scored_attn_prep_paged(const void *proj, int ld, int col0, const float *b_in, void *q_out, void *k_pool, void *v_pool,
                                const float *q_norm, const float *k_norm, float eps, const int *tok_seq, const int *tok_pos,
                                const int *block_table, int max_pages_per_seq, int tokens, int heads, int kv_heads, int dim, int vdim,
                                int rot_dims, float rot_base, int dtype, b200_stream_t stream) {
    B200_REQUIRE(proj && q_out && k_pool && v_pool && tok_seq && tok_pos && block_table, "scored_attn_prep: null pointer");
    B200_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && col0 >= 0 && ld >= col0 + (heads + kv_heads) * dim + kv_heads * vdim,
                 "scored_attn_prep: bad shape");
    B200_REQUIRE(rot_dims >= 0 && rot_dims <= dim && rot_dims % 2 == 0 && (rot_dims == 0 || rot_base > 0.0f), "scored_attn_prep: bad rotation");
    return launch_scored_prep(dtype, proj, ld, col0, b_in, q_out, k_pool, v_pool, q_norm, k_norm, eps, tok_seq, tok_pos, block_table,
                              max_pages_per_seq, tokens, heads, kv_heads, dim, vdim, rot_dims, rot_base, as_stream(stream));
}

int b200_scored_attention_paged(const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                                const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale,
                                const int *tok_seq, const int *tok_pos, const int *block_table, int max_pages_per_seq, int tokens, int heads,
                                int kv_heads, int dim, int vdim, float scale, int window, int attn_weight, int dtype, b200_stream_t stream) {
    B200_REQUIRE(q && k_pool && v_pool && out && tok_seq && tok_pos && block_table, "scored_attention: null pointer");
    B200_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && window >= 0 && out_ld >= heads * vdim,
                 "scored_attention: bad shape");
    B200_REQUIRE((dist_r1 == nullptr) == (dist_r2 == nullptr), "scored_attention: the distance penalty needs both of its vectors");
    const int max_keys = window > 0 ? std::min(window, max_pages_per_seq * kPageS) : max_pages_per_seq * kPageS;
    return launch_scored_attention(dtype, q, k_pool, v_pool, head_bias, dist_r1, dist_r2, gate_in, gate_ld, out, out_ld, out_scale, tok_seq, tok_pos,
                                   block_table, max_pages_per_seq, tokens, heads, kv_heads, dim, vdim, scale, window, attn_weight == B200_ATTN_SIGMOID,
                                   max_keys, as_stream(stream), nullptr);
}

int b200_scored_attention_tiles_paged(const void *q, const void *k_pool, const void *v_pool, const float *head_bias, const float *dist_r1,
                                      const float *dist_r2, const void *gate_in, int gate_ld, void *out, int out_ld, float out_scale,
                                      const int *tiles, int n_tiles, const int *block_table, int max_pages_per_seq, int heads, int kv_heads,
                                      int dim, int vdim, float scale, int window, int attn_weight, int dtype, b200_stream_t stream) {
    B200_REQUIRE(q && k_pool && v_pool && out && tiles && block_table, "scored_attention_tiles: null pointer");
    B200_REQUIRE(n_tiles >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && window >= 0, "scored_attention_tiles: bad shape");
    B200_REQUIRE(((uintptr_t)tiles & 15) == 0, "scored_attention_tiles: the tile list must be 16-byte aligned");
    return launch_scored_attention_tiles(dtype, q, k_pool, v_pool, head_bias, dist_r1, dist_r2, gate_in, gate_ld, out, out_ld, out_scale, tiles,
                                         n_tiles, block_table, max_pages_per_seq, heads, kv_heads, dim, vdim, scale, window,
                                         attn_weight == B200_ATTN_SIGMOID, as_stream(stream));
}
}
