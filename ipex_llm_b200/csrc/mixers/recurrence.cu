// Linear recurrences with a matrix state per head, and the short causal convolution that precedes one of them.
//
// Both recurrences act on every COLUMN of the state independently (a column = one value channel): with M [dim, vdim],
//   gated delta rule:        M <- g M;  u = beta (v - M^T k);  M <- M + k u^T;  o = M^T q
//   gated linear attention:  M <- diag(alpha) M + k v^T;       o = M^T q
// column j only needs k, q, the token's scalars and v_j.  So a column is owned by LPC lanes of a warp (LPC a power of two), each
// holding R rows of it in registers for the whole call; tokens are taken in order, their k / q (/ alpha) rows, scalars and
// v staged TC tokens at a time in shared memory by the whole block, unit norms and gates evaluated there in 32-bit floats.
// For the delta rule both dot products are taken on the state BEFORE the token's update,
//   a = M_old^T k,  c = M_old^T q:   u = beta (v - g a),   o = g c + (k . q) u,   M <- g M_old + k u^T,
// which is the same arithmetic reordered so that one round of shuffles serves both.
#include "mixers_common.cuh"

template <typename T>
__global__ void short_conv_silu_kernel(const T* __restrict__ proj, int B, int S, int ld, int off, int C, int taps, const T* __restrict__ w,
                                       const T* __restrict__ tail, T* __restrict__ tail_next, int slot0, const int32_t* __restrict__ pad,
                                       T* __restrict__ y) {
    long total = (long)B * S * C;
    const int tl = taps - 1 > 0 ? taps - 1 : 1;             // rows of a tail buffer
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        int c = (int)(i % C);
        long n = i / C;
        int b = (int)(n / S), t = (int)(n - (long)b * S);
        int first = pad ? pad[b] - slot0 : 0;                // new tokens before this index are padding
        if (first < 0) first = 0;
        auto input = [&](int tt) -> float {
            if (tt < 0) return to_f(tail[((long)b * tl + (taps - 1 + tt)) * C + c]);
            if (tt < first) return 0.0f;
            return to_f(proj[((long)b * S + tt) * ld + off + c]);
        };
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) acc += to_f(w[(long)c * taps + j]) * input(t - (taps - 1) + j);
        y[i] = from_f<T>(t < first ? 0.0f : silu_f(acc));
        if (t == S - 1)
            for (int r = 0; r < taps - 1; ++r) tail_next[((long)b * tl + r) * C + c] = from_f<T>(input(S - (taps - 1) + r));
    }
}

constexpr int REC_THREADS = 128;
constexpr int REC_TC = 16;                                  // tokens staged at a time (fewer for very wide heads)

struct RecArgs {
    const void* src;        // delta: conv output [B, S, C]; gla: projection [B, S, ld]
    int ld_src;
    int off_q, off_k, off_v;   // column offsets of head 0 inside a row of src
    int q_heads;            // heads of q / k (delta: kv_heads; gla: heads)
    const void* proj;       // delta: the projection that holds beta / decay logits
    int ld_proj, off_b, off_a;
    const void* A_log;
    const void* dt_bias;
    const void* z;          // gla: decay logits [B, S, heads * dim]
    float inv_tau;
    int B, S, heads, dim, vdim, slot0;
    const int32_t* pad;
    float* state;
    float* o;
    int lpc, tc;
};

template <typename T, int MODE, int R>                     // MODE 0: gated delta rule, 1: gated linear attention
__global__ void __launch_bounds__(REC_THREADS) linear_recurrence_kernel(RecArgs a) {
    extern __shared__ float sh[];
    const int lpc = a.lpc, dp = R * lpc, tc = a.tc;
    const int cols_blk = REC_THREADS / lpc;
    float* kbuf = sh;                                        // [tc][dp]
    float* qbuf = kbuf + tc * dp;                            // [tc][dp]
    float* abuf = qbuf + tc * dp;                            // [tc][dp] (gla only)
    float* vbuf = abuf + (MODE == 1 ? tc * dp : 0);          // [tc][cols_blk]
    float* sc = vbuf + tc * cols_blk;                        // [tc][4]: g, beta, k.q
    const int b = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int sub = tid % lpc;
    const int col_l = tid / lpc;
    const int col = blockIdx.x * cols_blk + col_l;
    const bool col_ok = col < a.vdim;
    const int dim = a.dim, vdim = a.vdim, S = a.S;
    const int qh = h / (a.heads / a.q_heads);
    const T* src = (const T*)a.src;

    float M[R];
    float* st = a.state + ((long)b * a.heads + h) * dim * vdim;
#pragma unroll
    for (int r = 0; r < R; ++r) {
        int i = r * lpc + sub;
        M[r] = (col_ok && i < dim) ? st[(long)i * vdim + col] : 0.0f;
    }
    int first = a.pad ? a.pad[b] - a.slot0 : 0;
    if (first < 0) first = 0;
    if (first > S) first = S;
    float* obase = a.o + (((long)b * S) * a.heads + h) * vdim;
    if (sub == 0 && col_ok)
        for (int t = 0; t < first; ++t) obase[(long)t * a.heads * vdim + col] = 0.0f;
    const float q_scale = rsqrtf((float)dim);

    for (int t0 = first; t0 < S; t0 += tc) {
        const int nt = S - t0 < tc ? S - t0 : tc;
        __syncthreads();
        // ---- stage nt tokens: a warp per token
        for (int tt = wid; tt < nt; tt += REC_THREADS / 32) {
            const T* row = src + ((long)b * S + t0 + tt) * a.ld_src;
            const T* qr = row + a.off_q + qh * dim;
            const T* kr = row + a.off_k + qh * dim;
            float sq = 0.0f, sk = 0.0f, skq = 0.0f;
            for (int i = lane; i < dp; i += 32) {
                float qv = i < dim ? to_f(qr[i]) : 0.0f, kv = i < dim ? to_f(kr[i]) : 0.0f;
                qbuf[tt * dp + i] = qv;
                kbuf[tt * dp + i] = kv;
                sq += qv * qv; sk += kv * kv; skq += qv * kv;
            }
            if (MODE == 0) {
                sq = warp_sum(sq); sk = warp_sum(sk); skq = warp_sum(skq);
                const float nq = q_scale / sqrtf(sq + 1e-6f), nk = 1.0f / sqrtf(sk + 1e-6f);
                __syncwarp();
                for (int i = lane; i < dp; i += 32) { qbuf[tt * dp + i] *= nq; kbuf[tt * dp + i] *= nk; }
                if (lane == 0) {
                    const T* pr = (const T*)a.proj + ((long)b * S + t0 + tt) * a.ld_proj;
                    float beta = sigmoid_f(to_f(pr[a.off_b + h]));
                    float dt = softplus_f(to_f(pr[a.off_a + h]) + to_f(((const T*)a.dt_bias)[h]));
                    sc[tt * 4 + 0] = expf(-expf(to_f(((const T*)a.A_log)[h])) * dt);
                    sc[tt * 4 + 1] = beta;
                    sc[tt * 4 + 2] = skq * nq * nk;
                }
            } else {
                const T* zr = (const T*)a.z + ((long)b * S + t0 + tt) * ((long)a.heads * dim) + h * dim;
                for (int i = lane; i < dp; i += 32) {
                    qbuf[tt * dp + i] *= q_scale;
                    abuf[tt * dp + i] = i < dim ? expf(log_sigmoid_f(to_f(zr[i])) * a.inv_tau) : 1.0f;
                }
            }
        }
        for (int i = tid; i < nt * cols_blk; i += REC_THREADS) {
            int tt = i / cols_blk, cl = i - tt * cols_blk;
            int cg = blockIdx.x * cols_blk + cl;
            vbuf[i] = cg < vdim ? to_f(src[((long)b * S + t0 + tt) * a.ld_src + a.off_v + h * vdim + cg]) : 0.0f;
        }
        __syncthreads();
        // ---- the tokens in order; a column's lanes only talk to each other
        for (int tt = 0; tt < nt; ++tt) {
            const float* kk = kbuf + tt * dp + sub;
            const float* qq = qbuf + tt * dp + sub;
            const float v = vbuf[tt * cols_blk + col_l];
            float o;
            if (MODE == 0) {
                float ak = 0.0f, cq = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { ak += M[r] * kk[r * lpc]; cq += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) { ak += __shfl_xor_sync(0xffffffffu, ak, m); cq += __shfl_xor_sync(0xffffffffu, cq, m); }
                const float g = sc[tt * 4 + 0], beta = sc[tt * 4 + 1], kq = sc[tt * 4 + 2];
                const float u = beta * (v - g * ak);
                o = g * cq + kq * u;
#pragma unroll
                for (int r = 0; r < R; ++r) M[r] = g * M[r] + kk[r * lpc] * u;
            } else {
                const float* aa = abuf + tt * dp + sub;
                o = 0.0f;
#pragma unroll
                for (int r = 0; r < R; ++r) { M[r] = aa[r * lpc] * M[r] + kk[r * lpc] * v; o += M[r] * qq[r * lpc]; }
                for (int m = lpc >> 1; m > 0; m >>= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
            }
            if (sub == 0 && col_ok) obase[(long)(t0 + tt) * a.heads * vdim + col] = o;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int i = r * lpc + sub;
            if (i < dim) st[(long)i * vdim + col] = M[r];
        }
    }
}

template <typename T, int MODE>
static int launch_recurrence(RecArgs a, cudaStream_t stream) {
    int r = a.dim <= 512 ? 16 : 32;
    int need = (a.dim + r - 1) / r;
    int lpc = 1;
    while (lpc < need) lpc <<= 1;
    if (lpc > 32) return (int)cudaErrorInvalidValue;         // heads wider than 1024 rows are not served
    int dp = r * lpc, cols_blk = REC_THREADS / lpc;
    int arrays = MODE == 1 ? 3 : 2;
    int tc = REC_TC;
    auto bytes = [&](int n) { return (size_t)n * (arrays * dp + cols_blk + 4) * sizeof(float); };
    while (tc > 1 && bytes(tc) > 40 * 1024) tc >>= 1;
    if (bytes(tc) > 48 * 1024) return (int)cudaErrorInvalidValue;
    a.lpc = lpc; a.tc = tc;
    dim3 grid((a.vdim + cols_blk - 1) / cols_blk, a.heads, a.B);
    if (r == 16) linear_recurrence_kernel<T, MODE, 16><<<grid, REC_THREADS, bytes(tc), stream>>>(a);
    else linear_recurrence_kernel<T, MODE, 32><<<grid, REC_THREADS, bytes(tc), stream>>>(a);
    return mixers_status();
}

extern "C" int mixers_short_conv_silu(int dtype, const void* proj, int B, int S, int ld, int off, int C, int taps, const void* w,
                                      const void* tail, void* tail_next, int slot0, const int32_t* pad, void* y, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (taps < 1) return (int)cudaErrorInvalidValue;
    long total = (long)B * S * C;
    long g = (total + 255) / 256;
    int blocks = (int)(g > 148L * 32 ? 148L * 32 : g);
    MIXERS_DISPATCH(dtype, short_conv_silu_kernel<T><<<blocks, 256, 0, (cudaStream_t)stream>>>((const T*)proj, B, S, ld, off, C, taps, (const T*)w,
                                                                                                 (const T*)tail, (T*)tail_next, slot0, pad, (T*)y));
    return mixers_status();
}

extern "C" int mixers_gated_delta_rule(int dtype, const void* conv, int B, int S, int kv_heads, int heads, int dim, int vdim,
                                       const void* proj, int ld, int off_b, int off_a, const void* A_log, const void* dt_bias, float* state,
                                       int slot0, const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    if (heads % kv_heads != 0) return (int)cudaErrorInvalidValue;
    RecArgs a = {};
    a.src = conv; a.ld_src = 2 * kv_heads * dim + heads * vdim;
    a.off_q = 0; a.off_k = kv_heads * dim; a.off_v = 2 * kv_heads * dim; a.q_heads = kv_heads;
    a.proj = proj; a.ld_proj = ld; a.off_b = off_b; a.off_a = off_a; a.A_log = A_log; a.dt_bias = dt_bias;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 0>(a, (cudaStream_t)stream)));
    return 0;
}

extern "C" int mixers_gated_linear_attention(int dtype, const void* proj, int B, int S, int ld, int heads, int dim, int vdim, const void* z,
                                             float tau, float* state, int slot0, const int32_t* pad, float* o, mixers_stream_t stream) {
    if (B <= 0 || S <= 0) return 0;
    RecArgs a = {};
    a.src = proj; a.ld_src = ld; a.off_q = 0; a.off_k = heads * dim; a.off_v = 2 * heads * dim; a.q_heads = heads;
    a.z = z; a.inv_tau = 1.0f / tau;
    a.B = B; a.S = S; a.heads = heads; a.dim = dim; a.vdim = vdim; a.slot0 = slot0; a.pad = pad; a.state = state; a.o = o;
    MIXERS_DISPATCH(dtype, return (launch_recurrence<T, 1>(a, (cudaStream_t)stream)));
    return 0;
}
