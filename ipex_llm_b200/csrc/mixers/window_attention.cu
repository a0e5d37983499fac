// Sliding-window attention whose weights are sigmoids of the scores (no softmax: nothing is normalised over the keys, so
// there is no running maximum and no rescaling, and a key's contribution is independent of every other key's).
//   window_qk_prepare: per-head RMS norm + rotation of interleaved pairs + the cache write, one launch for q, k and v;
//   sigmoid_window_attention: scores, sigmoid and the weighted sum of values in 32-bit floats straight from the cache.
#include "mixers_common.cuh"

// one warp per (token, head slot): slots [0, heads) are query heads, [heads, heads + kv) key heads, then kv value heads
template <typename T>
__global__ void window_qk_prepare_kernel(const T* __restrict__ proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                                         int dim, int vdim, const T* __restrict__ q_w, const T* __restrict__ k_w, float eps,
                                         const double* __restrict__ inv_freq, int rot_dims, float* __restrict__ q_out, T* __restrict__ k_store,
                                         T* __restrict__ v_store, int cap, int held, int shift, const int32_t* __restrict__ pad,
                                         const int32_t* __restrict__ dyn) {
    if (dyn) held = dyn[0];                                 // the length lives on the device when the step is replayed from a graph
    const int slots = heads + 2 * kv_heads;
    long warp = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    if (warp >= (long)B * S * slots) return;
    long n = warp / slots;
    int hs = (int)(warp - n * slots);
    int b = (int)(n / S), t = (int)(n - (long)b * S);
    int pos = held + t + shift - pad[b];                    // position in the sequence; negative = padding
    const T* row = proj + n * (long)ld;
    if (hs >= heads + kv_heads) {                           // a value head: copy
        int g = hs - heads - kv_heads;
        const T* src = row + off_v + g * vdim;
        T* dst = v_store + (((long)b * kv_heads + g) * cap + held + t) * vdim;
        for (int c = lane; c < vdim; c += 32) dst[c] = pos >= 0 ? src[c] : from_f<T>(0.0f);
        return;
    }
    const bool is_q = hs < heads;
    const int g = is_q ? hs : hs - heads;
    const T* src = row + (is_q ? off_q : off_k) + g * dim;
    const T* w = is_q ? q_w : k_w;
    float ss = 0.0f;
    for (int c = lane; c < dim; c += 32) { float v = to_f(src[c]); ss += v * v; }
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)dim + eps);
    float* qdst = is_q ? q_out + (n * heads + g) * (long)dim : nullptr;
    T* kdst = is_q ? nullptr : k_store + (((long)b * kv_heads + g) * cap + held + t) * dim;
    const double dpos = (double)pos;
    for (int p = lane; 2 * p < dim; p += 32) {
        int e0 = 2 * p, e1 = e0 + 1;
        float u = to_f(src[e0]) * inv * to_f(w[e0]);
        float v = e1 < dim ? to_f(src[e1]) * inv * to_f(w[e1]) : 0.0f;
        if (e0 < rot_dims) {                                // rot_dims is even: e1 is inside too
            // the angle and its sine / cosine in double precision (a handful per head and token): at position 10^3 a 32-bit
            // product position x frequency is already 6e-5 rad off
            double dsn, dcs;
            sincos(dpos * inv_freq[p], &dsn, &dcs);
            const float sn = (float)dsn, cs = (float)dcs;
            float ru = u * cs - v * sn, rv = v * cs + u * sn;
            u = ru; v = rv;
        }
        if (pos < 0) { u = 0.0f; v = 0.0f; }
        if (is_q) { qdst[e0] = u; if (e1 < dim) qdst[e1] = v; }
        else { kdst[e0] = from_f<T>(u); if (e1 < dim) kdst[e1] = from_f<T>(v); }
    }
}

// ---- the general kernel: any sizes, any dtype, 32-bit arithmetic throughout (the path of float32 models and of decoding).
// A block of ATT_WARPS warps per (token, query head); the warps take the visible keys in turns of 32.  Scores: a lane per key;
// the weighted sum: a lane per value column (columns lane, lane + 32, ...; up to VCOLS * 32 columns a pass), the keys' weights
// handed round by shuffles; the warps' partial sums meet in shared memory and are added in warp order.
constexpr int ATT_WARPS = 8;
constexpr int VCOLS = 8;

template <typename T>
__global__ void __launch_bounds__(ATT_WARPS * 32) sigmoid_window_attention_kernel(
        const float* __restrict__ q, const T* __restrict__ k_store, const T* __restrict__ v_store, int B, int S, int heads, int kv_heads, int dim,
        int vdim, int cap, int held, int shift, const int32_t* __restrict__ pad, int window, float scale, const T* __restrict__ head_bias,
        T* __restrict__ out, int ld_out, int out_col, float out_scale, const int32_t* __restrict__ dyn) {
    extern __shared__ float att_sh[];                       // q [dim], then partial sums [ATT_WARPS][VCOLS * 32]
    float* qs = att_sh;
    float* part = att_sh + dim;
    if (dyn) held = dyn[0];
    const int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = blockIdx.x;                           // (token, head)
    const long n = item / heads;
    const int h = (int)(item - n * heads);
    const int b = (int)(n / S), t = (int)(n - (long)b * S);
    const int g = h / (heads / kv_heads);
    const int c = held + t;                                 // the query's own storage index
    T* dst = out + n * (long)ld_out + out_col + h * vdim;
    const int first_real = pad[b] - shift;                  // storage index of the row's first real token (may be < 0)
    if (c < first_real) {
        for (int col = threadIdx.x; col < vdim; col += blockDim.x) dst[col] = from_f<T>(0.0f);
        return;
    }
    int lo = c - window + 1;
    if (lo < first_real) lo = first_real;
    if (lo < 0) lo = 0;
    const float* qsrc = q + item * (long)dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) qs[d] = qsrc[d];
    __syncthreads();
    const T* kbase = k_store + ((long)b * kv_heads + g) * cap * dim;
    const T* vbase = v_store + ((long)b * kv_heads + g) * cap * vdim;
    const float bias = to_f(head_bias[h]);
    // 16-bit values in rows that start on 16-byte boundaries: a lane owns 8 neighbouring columns (one 16-byte load a key), the
    // two halves of the warp take the even and the odd keys of a turn and meet at the end; 128 columns a pass
    const bool wide = sizeof(T) == 2 && (vdim & 7) == 0;
    for (int col0 = 0; wide && col0 < vdim; col0 += 128) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        const int mycol = col0 + (lane & 15) * 8;
        const int half = lane >> 4;
        for (int j0 = lo + 32 * wid; j0 <= c; j0 += 32 * ATT_WARPS) {
            const int j = j0 + lane;
            float wgt = 0.0f;
            if (j <= c) wgt = sigmoid_f(dot_row(qs, kbase + (long)j * dim, dim) * scale + bias);
            const int nk = c - j0 + 1 < 32 ? c - j0 + 1 : 32;
            for (int jj = 0; jj < nk; jj += 2) {             // keys past the end carry weight 0; their row index is clamped
                const int mine = jj + half;
                const float wj = __shfl_sync(0xffffffffu, wgt, mine & 31);
                if (mycol < vdim) {
                    const int row = j0 + mine <= c ? j0 + mine : c;
                    uint4 v = *reinterpret_cast<const uint4*>(vbase + (long)row * vdim + mycol);
                    const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += wj * to_f(e[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
        if (lane < 16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) part[wid * 128 + lane * 8 + i] = acc[i];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < 128; e += blockDim.x) {
            const int col = col0 + e;
            if (col < vdim) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < ATT_WARPS; ++w) sum += part[w * 128 + e];
                dst[col] = from_f<T>(sum * out_scale);
            }
        }
        __syncthreads();
    }
    for (int col0 = 0; !wide && col0 < vdim; col0 += VCOLS * 32) {
        float acc[VCOLS];
#pragma unroll
        for (int i = 0; i < VCOLS; ++i) acc[i] = 0.0f;
        for (int j0 = lo + 32 * wid; j0 <= c; j0 += 32 * ATT_WARPS) {
            const int j = j0 + lane;
            float wgt = 0.0f;
            if (j <= c) wgt = sigmoid_f(dot_row(qs, kbase + (long)j * dim, dim) * scale + bias);
            const int nk = c - j0 + 1 < 32 ? c - j0 + 1 : 32;
            for (int jj = 0; jj < nk; ++jj) {
                const float wj = __shfl_sync(0xffffffffu, wgt, jj);
                const T* vr = vbase + (long)(j0 + jj) * vdim + col0;
#pragma unroll
                for (int i = 0; i < VCOLS; ++i) {
                    const int col = lane + 32 * i;
                    if (col0 + col < vdim) acc[i] += wj * to_f(vr[col]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < VCOLS; ++i) part[(wid * VCOLS + i) * 32 + lane] = acc[i];
        __syncthreads();
        for (int e = threadIdx.x; e < VCOLS * 32; e += blockDim.x) {
            const int col = col0 + (e >> 5) * 32 + (e & 31);
            if (col < vdim) {
                float sum = 0.0f;
#pragma unroll
                for (int w = 0; w < ATT_WARPS; ++w) sum += part[w * VCOLS * 32 + e];
                dst[col] = from_f<T>(sum * out_scale);
            }
        }
        __syncthreads();
    }
}

// ---- many new tokens of a 16-bit model: both products on the tensor cores (mma.sync m16n8k16, 32-bit accumulators).
// A block of 4 warps takes 64 consecutive query tokens of one head (16 rows a warp, their queries rounded to 16 bits in
// registers) and walks the keys they can see 32 at a time: K and V tiles staged in shared memory (rows padded by 16 bytes so
// that the fragment reads and the transposing ldmatrix are free of bank conflicts), S = Q K^T, P = sigmoid(S scale + bias)
// in 32-bit floats with everything outside a row's window set to zero, then O += P V.  There is no softmax, hence no running
// maximum and no rescaling of O.  P goes to the tensor cores as the sum of two 16-bit numbers (its rounding and the
// rounding's remainder), so the weights keep ~16 bits of mantissa instead of 8.
template <typename T> struct Mma16;
template <> struct Mma16<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u)); }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Mma16<__half> {
    static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
        __half2 v = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&v);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t u) { return __half22float2(*reinterpret_cast<__half2*>(&u)); }
    static __device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

constexpr int TC_ROWS = 64, TC_KEYS = 32;

template <typename T, int KDMAX, int NDMAX>                // dim <= 16 KDMAX, vdim <= 8 NDMAX; both multiples of 16
__global__ void __launch_bounds__(128) sigmoid_window_attention_tc_kernel(
        const float* __restrict__ q, const T* __restrict__ k_store, const T* __restrict__ v_store, int B, int S, int heads, int kv_heads, int dim,
        int vdim, int cap, int held, int shift, const int32_t* __restrict__ pad, int window, float scale, const T* __restrict__ head_bias,
        T* __restrict__ out, int ld_out, int out_col, float out_scale) {
    extern __shared__ __align__(16) unsigned char tc_sh[];
    const int kstride = dim + 8, vstride = vdim + 8;        // elements
    T* Ks = reinterpret_cast<T*>(tc_sh);                    // [TC_KEYS][kstride]
    T* Vs = Ks + TC_KEYS * kstride;                         // [TC_KEYS][vstride]
    const int b = blockIdx.z, h = blockIdx.y, t0 = blockIdx.x * TC_ROWS;
    const int g = h / (heads / kv_heads);
    const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31, gr = lane >> 2, tq = lane & 3;
    const int kdn = dim >> 4, ndn = vdim >> 3;
    const int first_real = pad[b] - shift;
    const int t_last = (t0 + TC_ROWS - 1 < S - 1) ? t0 + TC_ROWS - 1 : S - 1;
    const int c_hi = held + t_last;                         // newest key this block can see (initialised storage ends here)
    int j_start = held + t0 - window + 1;
    if (j_start < first_real) j_start = first_real;
    if (j_start < 0) j_start = 0;
    // this warp's rows
    const int r0 = t0 + wid * 16;
    const int tr[2] = {r0 + gr, r0 + gr + 8};
    int row_c[2], row_lo[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        row_c[i] = held + tr[i];
        int lo = row_c[i] - window + 1;
        if (lo < first_real) lo = first_real;
        if (lo < 0) lo = 0;
        row_lo[i] = lo;
        if (tr[i] >= S || row_c[i] < first_real) { row_c[i] = -1; row_lo[i] = 0; }      // nothing visible
    }
    const int warp_hi = held + ((r0 + 15 < S - 1) ? r0 + 15 : S - 1);
    int warp_lo = held + r0 - window + 1;
    // queries -> A fragments
    uint32_t qa[KDMAX][4];
#pragma unroll
    for (int kd = 0; kd < KDMAX; ++kd) {
#pragma unroll
        for (int i = 0; i < 4; ++i) qa[kd][i] = 0u;
        if (kd < kdn) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                if (tr[i] < S) {
                    const float* src = q + (((long)b * S + tr[i]) * heads + h) * dim + kd * 16 + 2 * tq;
                    float2 lo2 = *reinterpret_cast<const float2*>(src), hi2 = *reinterpret_cast<const float2*>(src + 8);
                    qa[kd][i] = Mma16<T>::pack(lo2.x, lo2.y);
                    qa[kd][2 + i] = Mma16<T>::pack(hi2.x, hi2.y);
                }
            }
        }
    }
    float oacc[NDMAX][4];
#pragma unroll
    for (int nd = 0; nd < NDMAX; ++nd)
#pragma unroll
        for (int i = 0; i < 4; ++i) oacc[nd][i] = 0.0f;
    const float bias = to_f(head_bias[h]);
    const T* kbase = k_store + ((long)b * kv_heads + g) * cap * dim;
    const T* vbase = v_store + ((long)b * kv_heads + g) * cap * vdim;
    const int kchunks = dim >> 3, vchunks = vdim >> 3;      // 16-byte pieces per row

    for (int jt = j_start; jt <= c_hi; jt += TC_KEYS) {
        __syncthreads();                                    // the previous tile has been consumed
        for (int id = tid; id < TC_KEYS * kchunks; id += 128) {
            int r = id / kchunks, cch = id - r * kchunks;
            int j = jt + r <= c_hi ? jt + r : c_hi;         // rows past the end repeat the last one (their weights are zero)
            *reinterpret_cast<uint4*>(Ks + r * kstride + cch * 8) = *reinterpret_cast<const uint4*>(kbase + (long)j * dim + cch * 8);
        }
        for (int id = tid; id < TC_KEYS * vchunks; id += 128) {
            int r = id / vchunks, cch = id - r * vchunks;
            int j = jt + r <= c_hi ? jt + r : c_hi;
            *reinterpret_cast<uint4*>(Vs + r * vstride + cch * 8) = *reinterpret_cast<const uint4*>(vbase + (long)j * vdim + cch * 8);
        }
        __syncthreads();
        if (jt > warp_hi || jt + TC_KEYS - 1 < warp_lo) continue;        // no row of this warp sees the tile
        // S = Q K^T for 16 rows x 32 keys
        float sc[4][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int i = 0; i < 4; ++i) sc[nt][i] = 0.0f;
            const T* krow = Ks + (nt * 8 + gr) * kstride + 2 * tq;
#pragma unroll
            for (int kd = 0; kd < KDMAX; ++kd) {
                if (kd < kdn) {
                    uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + kd * 16);
                    uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + kd * 16 + 8);
                    Mma16<T>::mma(sc[nt], qa[kd], b0, b1);
                }
            }
        }
        // P = sigmoid(S scale + bias) inside each row's window, split into two 16-bit parts
        uint32_t ph[2][4], pl[2][4];
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            float p[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int j = jt + nt * 8 + 2 * tq + (i & 1);
                const int r = i >> 1;
                // hardware exponential and reciprocal (~2 ulp): these weights are split into two 16-bit parts right below,
                // the exact division of sigmoid_f would cost more than the tile's MMAs
                p[i] = (j >= row_lo[r] && j <= row_c[r]) ? __fdividef(1.0f, 1.0f + __expf(-(sc[nt][i] * scale + bias))) : 0.0f;
            }
            const int ks = nt >> 1, half = nt & 1;
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                uint32_t hi = Mma16<T>::pack(p[2 * r], p[2 * r + 1]);
                float2 back = Mma16<T>::unpack(hi);
                ph[ks][2 * half + r] = hi;
                pl[ks][2 * half + r] = Mma16<T>::pack(p[2 * r] - back.x, p[2 * r + 1] - back.y);
            }
        }
        // O += P V
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
            for (int np = 0; np < NDMAX / 2; ++np) {
                if (2 * np < ndn) {
                    uint32_t v0, v1, v2, v3;
                    const T* vaddr = Vs + (ks * 16 + (lane & 15)) * vstride + np * 16 + ((lane >> 4) << 3);
                    uint32_t sa = (uint32_t)__cvta_generic_to_shared(vaddr);
                    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                                 : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3) : "r"(sa));
                    Mma16<T>::mma(oacc[2 * np], ph[ks], v0, v1);
                    Mma16<T>::mma(oacc[2 * np], pl[ks], v0, v1);
                    Mma16<T>::mma(oacc[2 * np + 1], ph[ks], v2, v3);
                    Mma16<T>::mma(oacc[2 * np + 1], pl[ks], v2, v3);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        if (tr[i] < S) {
            T* dst = out + ((long)b * S + tr[i]) * ld_out + out_col + h * vdim + 2 * tq;
#pragma unroll
            for (int nd = 0; nd < NDMAX; ++nd) {
                if (nd < ndn) {
                    dst[nd * 8] = from_f<T>(oacc[nd][2 * i] * out_scale);
                    dst[nd * 8 + 1] = from_f<T>(oacc[nd][2 * i + 1] * out_scale);
                }
            }
        }
    }
}

template <typename T, int KDMAX, int NDMAX>
static int launch_attention_tc(const float* q, const void* k_store, const void* v_store, int B, int S, int heads, int kv_heads, int dim, int vdim,
                               int cap, int held, int shift, const int32_t* pad, int window, float scale, const void* head_bias, void* out,
                               int ld_out, int out_col, float out_scale, cudaStream_t stream) {
    size_t smem = (size_t)TC_KEYS * (dim + 8 + vdim + 8) * sizeof(T);
    dim3 grid((S + TC_ROWS - 1) / TC_ROWS, heads, B);
    sigmoid_window_attention_tc_kernel<T, KDMAX, NDMAX><<<grid, 128, smem, stream>>>(
        q, (const T*)k_store, (const T*)v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window, scale, (const T*)head_bias,
        (T*)out, ld_out, out_col, out_scale);
    return mixers_status();
}

template <typename T>
static int attention_tc(const float* q, const void* k_store, const void* v_store, int B, int S, int heads, int kv_heads, int dim, int vdim,
                        int cap, int held, int shift, const int32_t* pad, int window, float scale, const void* head_bias, void* out, int ld_out,
                        int out_col, float out_scale, cudaStream_t stream) {
#define TC_ARGS q, k_store, v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window, scale, head_bias, out, ld_out, out_col, out_scale, stream
    if (dim <= 64 && vdim <= 64) return launch_attention_tc<T, 4, 8>(TC_ARGS);
    if (dim <= 128 && vdim <= 128) return launch_attention_tc<T, 8, 16>(TC_ARGS);
    return launch_attention_tc<T, 16, 32>(TC_ARGS);
#undef TC_ARGS
}

extern "C" int mixers_window_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads,
                                        int kv_heads, int dim, int vdim, const void* q_w, const void* k_w, float eps, const double* inv_freq,
                                        int rot_dims, float* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                                        const int32_t* pad, const int32_t* dyn, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (held + S > cap || rot_dims > dim || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
    long warps = (long)B * S * (heads + 2 * kv_heads);
    int blocks = (int)((warps + 3) / 4);
    MIXERS_DISPATCH(dtype, window_qk_prepare_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>(
        (const T*)proj, B, S, ld, off_q, off_k, off_v, heads, kv_heads, dim, vdim, (const T*)q_w, (const T*)k_w, eps, inv_freq, rot_dims,
        q_out, (T*)k_store, (T*)v_store, cap, held, shift, pad, dyn));
    return mixers_status();
}

extern "C" int mixers_sigmoid_window_attention(int dtype, const float* q, const void* k_store, const void* v_store, int B, int S, int heads,
                                               int kv_heads, int dim, int vdim, int cap, int held, int shift, const int32_t* pad, int window,
                                               float scale, const void* head_bias, void* out, int ld_out, int out_col, float out_scale,
                                               const int32_t* dyn, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    size_t smem = ((size_t)dim + ATT_WARPS * VCOLS * 32) * sizeof(float);
    if (held + S > cap || window < 1 || heads % kv_heads != 0 || smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    // many new tokens of a 16-bit model with head sizes the fragments tile: the tensor-core kernel
    if (dtype != 0 && !dyn && S >= 16 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 256 && vdim <= 256) {
        if (dtype == 1) return attention_tc<__nv_bfloat16>(q, k_store, v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window,
                                                           scale, head_bias, out, ld_out, out_col, out_scale, (cudaStream_t)stream);
        if (dtype == 2) return attention_tc<__half>(q, k_store, v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window, scale,
                                                    head_bias, out, ld_out, out_col, out_scale, (cudaStream_t)stream);
    }
    long items = (long)B * S * heads;
    MIXERS_DISPATCH(dtype, sigmoid_window_attention_kernel<T><<<(unsigned)items, ATT_WARPS * 32, smem, (cudaStream_t)stream>>>(
        q, (const T*)k_store, (const T*)v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window, scale, (const T*)head_bias,
        (T*)out, ld_out, out_col, out_scale, dyn));
    return mixers_status();
}
