// Sliding-window attention whose weights are sigmoids of the scores (no softmax: nothing is normalised over the keys, so
// there is no running maximum and no rescaling, and a key's contribution is independent of every other key's).
//   window_qk_prepare: per-head RMS norm + rotation of interleaved pairs + the cache write, one launch for q, k and v;
//   sigmoid_window_attention: scores, sigmoid and the weighted sum of values in 32-bit floats straight from the cache.
#include "mixers_common.cuh"

// one warp per (token, head slot): slots [0, heads) are query heads, [heads, heads + kv) key heads, then kv value heads
template <typename T>
__global__ void window_qk_prepare_kernel(const T* __restrict__ proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads, int kv_heads,
                                         int dim, int vdim, const T* __restrict__ q_w, const T* __restrict__ k_w, float eps,
                                         const float* __restrict__ inv_freq, int rot_dims, float* __restrict__ q_out, T* __restrict__ k_store,
                                         T* __restrict__ v_store, int cap, int held, int shift, const int32_t* __restrict__ pad) {
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
    const float fpos = (float)pos;
    for (int p = lane; 2 * p < dim; p += 32) {
        int e0 = 2 * p, e1 = e0 + 1;
        float u = to_f(src[e0]) * inv * to_f(w[e0]);
        float v = e1 < dim ? to_f(src[e1]) * inv * to_f(w[e1]) : 0.0f;
        if (e0 < rot_dims) {                                // rot_dims is even: e1 is inside too
            float sn, cs;
            sincosf(fpos * inv_freq[p], &sn, &cs);
            float ru = u * cs - v * sn, rv = v * cs + u * sn;
            u = ru; v = rv;
        }
        if (pos < 0) { u = 0.0f; v = 0.0f; }
        if (is_q) { qdst[e0] = u; if (e1 < dim) qdst[e1] = v; }
        else { kdst[e0] = from_f<T>(u); if (e1 < dim) kdst[e1] = from_f<T>(v); }
    }
}

// One warp per (token, query head).  Scores: a lane per key, 32 keys at a time; the weighted sum: a lane per value column
// (columns lane, lane + 32, ...; up to VCOLS * 32 columns a pass), the keys' weights handed round by shuffles.
constexpr int ATT_WARPS = 4;
constexpr int VCOLS = 8;

template <typename T>
__global__ void sigmoid_window_attention_kernel(const float* __restrict__ q, const T* __restrict__ k_store, const T* __restrict__ v_store, int B, int S,
                                                int heads, int kv_heads, int dim, int vdim, int cap, int held, int shift,
                                                const int32_t* __restrict__ pad, int window, float scale, const T* __restrict__ head_bias,
                                                T* __restrict__ out, int ld_out, int out_col, float out_scale) {
    extern __shared__ float q_sh[];                         // [ATT_WARPS][dim]
    int wid = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long warp = blockIdx.x * (long)ATT_WARPS + wid;
    if (warp >= (long)B * S * heads) return;
    long n = warp / heads;
    int h = (int)(warp - n * heads);
    int b = (int)(n / S), t = (int)(n - (long)b * S);
    int g = h / (heads / kv_heads);
    int c = held + t;                                       // the query's own storage index
    T* dst = out + n * (long)ld_out + out_col + h * vdim;
    int first_real = pad[b] - shift;                        // storage index of the row's first real token (may be < 0)
    if (c < first_real) {
        for (int col = lane; col < vdim; col += 32) dst[col] = from_f<T>(0.0f);
        return;
    }
    int lo = c - window + 1;
    if (lo < first_real) lo = first_real;
    if (lo < 0) lo = 0;
    float* qs = q_sh + wid * dim;
    const float* qsrc = q + warp * (long)dim;
    for (int d = lane; d < dim; d += 32) qs[d] = qsrc[d];
    __syncwarp();
    const T* kbase = k_store + ((long)b * kv_heads + g) * cap * dim;
    const T* vbase = v_store + ((long)b * kv_heads + g) * cap * vdim;
    const float bias = to_f(head_bias[h]);
    for (int col0 = 0; col0 < vdim; col0 += VCOLS * 32) {
        float acc[VCOLS];
#pragma unroll
        for (int i = 0; i < VCOLS; ++i) acc[i] = 0.0f;
        for (int j0 = lo; j0 <= c; j0 += 32) {
            int j = j0 + lane;
            float wgt = 0.0f;
            if (j <= c) {
                const T* kr = kbase + (long)j * dim;
                float s = 0.0f;
                for (int d = 0; d < dim; ++d) s += qs[d] * to_f(kr[d]);
                wgt = sigmoid_f(s * scale + bias);
            }
            int nk = c - j0 + 1 < 32 ? c - j0 + 1 : 32;
            for (int jj = 0; jj < nk; ++jj) {
                float wj = __shfl_sync(0xffffffffu, wgt, jj);
                const T* vr = vbase + (long)(j0 + jj) * vdim + col0;
#pragma unroll
                for (int i = 0; i < VCOLS; ++i) {
                    int col = lane + 32 * i;
                    if (col0 + col < vdim) acc[i] += wj * to_f(vr[col]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < VCOLS; ++i) {
            int col = col0 + lane + 32 * i;
            if (col < vdim) dst[col] = from_f<T>(acc[i] * out_scale);
        }
    }
}

extern "C" int mixers_window_qk_prepare(int dtype, const void* proj, int B, int S, int ld, int off_q, int off_k, int off_v, int heads,
                                        int kv_heads, int dim, int vdim, const void* q_w, const void* k_w, float eps, const float* inv_freq,
                                        int rot_dims, float* q_out, void* k_store, void* v_store, int cap, int held, int shift,
                                        const int32_t* pad, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (held + S > cap || rot_dims > dim || (rot_dims & 1)) return (int)cudaErrorInvalidValue;
    long warps = (long)B * S * (heads + 2 * kv_heads);
    int blocks = (int)((warps + 3) / 4);
    MIXERS_DISPATCH(dtype, window_qk_prepare_kernel<T><<<blocks, 128, 0, (cudaStream_t)stream>>>(
        (const T*)proj, B, S, ld, off_q, off_k, off_v, heads, kv_heads, dim, vdim, (const T*)q_w, (const T*)k_w, eps, inv_freq, rot_dims,
        q_out, (T*)k_store, (T*)v_store, cap, held, shift, pad));
    return mixers_status();
}

extern "C" int mixers_sigmoid_window_attention(int dtype, const float* q, const void* k_store, const void* v_store, int B, int S, int heads,
                                               int kv_heads, int dim, int vdim, int cap, int held, int shift, const int32_t* pad, int window,
                                               float scale, const void* head_bias, void* out, int ld_out, int out_col, float out_scale,
                                               mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (held + S > cap || window < 1 || heads % kv_heads != 0 || (size_t)ATT_WARPS * dim * sizeof(float) > 48 * 1024) return (int)cudaErrorInvalidValue;
    long warps = (long)B * S * heads;
    int blocks = (int)((warps + ATT_WARPS - 1) / ATT_WARPS);
    size_t smem = (size_t)ATT_WARPS * dim * sizeof(float);
    MIXERS_DISPATCH(dtype, sigmoid_window_attention_kernel<T><<<blocks, ATT_WARPS * 32, smem, (cudaStream_t)stream>>>(
        q, (const T*)k_store, (const T*)v_store, B, S, heads, kv_heads, dim, vdim, cap, held, shift, pad, window, scale, (const T*)head_bias,
        (T*)out, ld_out, out_col, out_scale));
    return mixers_status();
}
