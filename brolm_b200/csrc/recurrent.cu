// Mixers that carry a state of fixed size from token to token instead of a cache of keys:
// a short causal convolution per channel, a gated diagonal recurrence (one number per channel),
// and a selective state space (a matrix of N x P numbers per head).
//
// A step's tokens are packed back to back; sequence b owns rows cu_q[b] .. cu_q[b+1], holds kv_len[b]
// tokens after the step and keeps its state in row slots[b] of a float tensor [slots][state_stride].
// The same kernels serve a prompt and a decode step (one token per sequence): a sequence's state is read
// at the start of its rows and written at their end, so how a sequence was cut into steps changes nothing
// but the rounding of sums that are made in the same order anyway.  A row b with kv_len[b] <= 0 is padding.
//
// Everything here is float arithmetic: the state, the decays and their exponentials, the gates, the
// step sizes.  Inputs come as float or bfloat16 (the projections' results), small vectors as float.
#include "common.cuh"

namespace {

enum : int { CONV_NONE = 0, CONV_SILU = 1 };

__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
}

struct SeqArgs {
    const int32_t* cu_q;      // [B + 1]
    const int32_t* kv_len;    // [B]
    const int32_t* slots;     // [B]
    float* state;             // [slots][state_stride]
    long state_stride;
};

// ---------------------------------------------------------------------------
// Causal convolution per channel over the packed tokens.
//   in(q, c)  = x[row of position q][c] + in_bias[c]         (q inside the step)
//             = tail[q - (first - (K-1))][c]                  (q before the step: the K-1 inputs the state keeps;
//                                                              zeros before the sequence's start)
//   out[t, c] = act(sum_j w[c][j] * in(pos - (K-1) + j, c) + bias[c])
// The tail is left as it is (conv_tail_kernel moves it on once everything that reads it has run).
// ---------------------------------------------------------------------------
template <typename X>
__global__ void __launch_bounds__(256) causal_conv_kernel(const X* __restrict__ x, long ldx, const float* __restrict__ in_bias,
                                                          const float* __restrict__ w, const float* __restrict__ bias, int C, int K,
                                                          int act, const int32_t* __restrict__ tok_seq,
                                                          const int32_t* __restrict__ positions, SeqArgs s, long tail_off,
                                                          float* __restrict__ out, long ldo) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int pos = positions[t];
    if (pos < 0 || c >= C) return;
    const int b = tok_seq[t];
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int first = s.kv_len[b] - q_len;
    const float* tail = s.state + (size_t)s.slots[b] * s.state_stride + tail_off;
    const float ib = in_bias ? in_bias[c] : 0.0f;
    float acc = bias ? bias[c] : 0.0f;
    pdl_wait();
    for (int j = 0; j < K; ++j) {
        const int q = pos - (K - 1) + j;
        float v;
        if (q >= first)
            v = to_float(x[(size_t)(q0 + q - first) * ldx + c]) + ib;
        else
            v = tail[(size_t)(q - first + K - 1) * C + c];
        acc = fmaf(w[(size_t)c * K + j], v, acc);
    }
    if (act == CONV_SILU) acc = acc / (1.0f + expf(-acc));
    out[(size_t)t * ldo + c] = acc;
}

// tail[k][c] <- in(new_len - (K-1) + k, c), k = 0 .. K-2, ascending: place k reads old place k + q_len, which
// is written later.
template <typename X>
__global__ void __launch_bounds__(256) conv_tail_kernel(const X* __restrict__ x, long ldx, const float* __restrict__ in_bias, int C,
                                                        int K, SeqArgs s, long tail_off) {
    pdl_trigger();
    const int b = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int kv_len = s.kv_len[b];
    if (kv_len <= 0 || c >= C) return;
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int first = kv_len - q_len;
    float* tail = s.state + (size_t)s.slots[b] * s.state_stride + tail_off;
    const float ib = in_bias ? in_bias[c] : 0.0f;
    pdl_wait();
    for (int k = 0; k < K - 1; ++k) {
        const int q = kv_len - (K - 1) + k;
        float v;
        if (q >= first)
            v = to_float(x[(size_t)(q0 + q - first) * ldx + c]) + ib;
        else
            v = tail[(size_t)(q - first + K - 1) * C + c];
        tail[(size_t)k * C + c] = v;
    }
}

// ---------------------------------------------------------------------------
// Gated diagonal recurrence.  Per channel c of block c / bs:
//   r = sigmoid(pre[t][blk][0][o] + rb[c]),  i = sigmoid(pre[t][blk][1][o] + ib[c])       (pre: the block-diagonal
//   log a = -decay_scale * r * softplus(lam[c]),  a = exp(log a)                            products of u, made before)
//   S <- a S + sqrt(1 - a^2) * i * u[t][c];   out[t][c] = S * gelu_tanh(y_raw[t][c] + yb[c])
// 1 - a^2 is taken as -expm1(2 log a) and a S as S + expm1(log a) S, which keep their digits when a is close to
// one (a state that remembers for thousands of tokens): a itself, rounded to float, would not.
// ---------------------------------------------------------------------------
template <typename Y, typename O>
__global__ void __launch_bounds__(128) gated_scan_kernel(const float* __restrict__ pre, long ldpre, const float* __restrict__ u,
                                                         long ldu, const Y* __restrict__ y_raw, long ldy,
                                                         const float* __restrict__ yb, const float* __restrict__ rb,
                                                         const float* __restrict__ ib, const float* __restrict__ lam,
                                                         float decay_scale, int width, int bs, SeqArgs s, O* __restrict__ out,
                                                         long ldo) {
    pdl_trigger();
    const int b = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int kv_len = s.kv_len[b];
    if (kv_len <= 0 || c >= width) return;
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int blk = c / bs, o = c - blk * bs;
    const size_t pr = (size_t)blk * 2 * bs + o, pi = pr + bs;
    const float sp = -decay_scale * softplus_f(lam[c]);
    const float bias_r = rb[c], bias_i = ib[c], bias_y = yb ? yb[c] : 0.0f;
    float* st = s.state + (size_t)s.slots[b] * s.state_stride + c;
    pdl_wait();
    float S = *st;
    constexpr int U = 4;
    for (int t0 = 0; t0 < q_len; t0 += U) {
        float vr[U], vi[U], vu[U], vy[U];
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t0 + k < q_len) {
                const size_t row = (size_t)(q0 + t0 + k);
                vr[k] = pre[row * ldpre + pr];
                vi[k] = pre[row * ldpre + pi];
                vu[k] = u[row * ldu + c];
                vy[k] = to_float(y_raw[row * ldy + c]);
            }
        }
#pragma unroll
        for (int k = 0; k < U; ++k) {
            if (t0 + k < q_len) {
                const float r = sigmoid_f(vr[k] + bias_r), g = sigmoid_f(vi[k] + bias_i);
                const float log_a = sp * r;
                const float drive = sqrtf(-expm1f(2.0f * log_a)) * g * vu[k];
                S = fmaf(expm1f(log_a), S, S) + drive;          // a S as S + (a - 1) S
                out[(size_t)(q0 + t0 + k) * ldo + c] = from_float<O>(S * gelu_tanh_f(vy[k] + bias_y));
            }
        }
    }
    *st = S;
}

// ---------------------------------------------------------------------------
// Selective state space.  Per head h (group g = h / (heads / groups)), S of N x P floats, kept as [h][p][n]:
//   dt = softplus(dt_raw[t][h] + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt * B[t][g] x[t][h]^T
//   y[t][h] = S^T C[t][g] + D[h] x[t][h]
// xbc row t: [ x: heads*P | B: groups*N | C: groups*N ] float (after the convolution and its activation).
// A block takes one (sequence, head) and a run of P / (128 / nsplit) values of p; thread (p, s) keeps the
// states n = s + nsplit * j, j < NPT, in registers.  The tokens of a sequence are staged sixteen at a time.
// ---------------------------------------------------------------------------
constexpr int SSM_TC = 16;

template <typename X, int NPT>
__global__ void __launch_bounds__(128) ssm_scan_kernel(const float* __restrict__ xbc, long ldx, const X* __restrict__ dt_raw, long lddt,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                       const float* __restrict__ Dv, int heads, int groups, int P, int N,
                                                       int nsplit, SeqArgs s, float* __restrict__ y, long ldy) {
    extern __shared__ float sm[];
    pdl_trigger();
    const int VT = 128 / nsplit;
    float* sB = sm;                         // [TC][N]
    float* sC = sB + SSM_TC * N;            // [TC][N]
    float* sx = sC + SSM_TC * N;            // [TC][VT]
    float* sdt = sx + SSM_TC * VT;          // [TC]
    float* sdec = sdt + SSM_TC;             // [TC]
    const int b = blockIdx.z, h = blockIdx.y, g = h / (heads / groups);
    const int kv_len = s.kv_len[b];
    if (kv_len <= 0) return;
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int sl = threadIdx.x % nsplit, vi = threadIdx.x / nsplit;
    const int p0 = blockIdx.x * VT, p = p0 + vi;
    const bool p_ok = p < P;
    const float A = -expf(A_log[h]), D = Dv[h], dtb = dt_bias[h];
    float* st = s.state + (size_t)s.slots[b] * s.state_stride + ((size_t)h * P + (p_ok ? p : 0)) * N;
    const int inner = heads * P;
    const size_t offB = (size_t)inner + (size_t)g * N, offC = (size_t)inner + (size_t)(groups + g) * N;
    pdl_wait();
    float S[NPT];
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
        const int n = sl + nsplit * j;
        S[j] = (p_ok && n < N) ? st[n] : 0.0f;
    }
    for (int t0 = 0; t0 < q_len; t0 += SSM_TC) {
        const int n_tok = min(SSM_TC, q_len - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_tok * N; idx += 128) {
            const int tt = idx / N, n = idx - tt * N;
            const float* row = xbc + (size_t)(q0 + t0 + tt) * ldx;
            sB[tt * N + n] = row[offB + n];
            sC[tt * N + n] = row[offC + n];
        }
        for (int idx = threadIdx.x; idx < n_tok * VT; idx += 128) {
            const int tt = idx / VT, v = idx - tt * VT;
            sx[tt * VT + v] = (p0 + v < P) ? xbc[(size_t)(q0 + t0 + tt) * ldx + (size_t)h * P + p0 + v] : 0.0f;
        }
        if (threadIdx.x < n_tok) {
            const float dt = softplus_f(to_float(dt_raw[(size_t)(q0 + t0 + threadIdx.x) * lddt + h]) + dtb);
            sdt[threadIdx.x] = dt;
            sdec[threadIdx.x] = expm1f(A * dt);            // decay - 1: the decay is applied as S + (decay - 1) S
        }
        __syncthreads();
        for (int tt = 0; tt < n_tok; ++tt) {
            const float dt = sdt[tt], dec = sdec[tt], xv = sx[tt * VT + vi];
            const float dx = dt * xv;
            const float* rb = sB + tt * N;
            const float* rc = sC + tt * N;
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < NPT; ++j) {
                const int n = sl + nsplit * j;
                if (n < N) {
                    S[j] = fmaf(dec, S[j], S[j]) + dx * rb[n];
                    acc = fmaf(S[j], rc[n], acc);
                }
            }
            for (int o = nsplit >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (sl == 0 && p_ok) y[(size_t)(q0 + t0 + tt) * ldy + (size_t)h * P + p] = fmaf(D, xv, acc);
        }
    }
    if (p_ok) {
#pragma unroll
        for (int j = 0; j < NPT; ++j) {
            const int n = sl + nsplit * j;
            if (n < N) st[n] = S[j];
        }
    }
}

SeqArgs seq_args(const void* cu_q, const void* kv_len, const void* slots, void* state, long state_stride) {
    SeqArgs s;
    s.cu_q = (const int32_t*)cu_q; s.kv_len = (const int32_t*)kv_len; s.slots = (const int32_t*)slots;
    s.state = (float*)state; s.state_stride = state_stride;
    return s;
}

}  // namespace

// out [tokens, C] float = act(conv(x + in_bias) + bias); x float or bfloat16 with ldx elements between rows.
BROLM_API int brolm_causal_conv(const void* x, int x_dtype, long ldx, const void* in_bias, const void* w, const void* bias,
                                int C, int K, int act, const void* tok_seq, const void* positions, const void* cu_q,
                                const void* kv_len, const void* slots, void* state, long state_stride, long tail_off,
                                void* out, long ldo, int tokens, cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (C <= 0 || K <= 0 || (act != CONV_NONE && act != CONV_SILU)) return BROLM_ERR_BAD_SIZE;
    if ((C + 255) / 256 > 65535) return BROLM_ERR_TOO_LARGE;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid(tokens, (C + 255) / 256);
    if (x_dtype == BROLM_F32)
        return launch_pdl(causal_conv_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ldx, (const float*)in_bias,
                          (const float*)w, (const float*)bias, C, K, act, (const int32_t*)tok_seq, (const int32_t*)positions, s,
                          tail_off, (float*)out, ldo);
    if (x_dtype == BROLM_BF16)
        return launch_pdl(causal_conv_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, (const float*)in_bias,
                          (const float*)w, (const float*)bias, C, K, act, (const int32_t*)tok_seq, (const int32_t*)positions, s,
                          tail_off, (float*)out, ldo);
    return BROLM_ERR_BAD_DTYPE;
}

// The state's K-1 kept inputs of every sequence moved on by the step's tokens.  Runs after everything that reads them.
BROLM_API int brolm_conv_tail(const void* x, int x_dtype, long ldx, const void* in_bias, int C, int K, const void* cu_q,
                              const void* kv_len, const void* slots, void* state, long state_stride, long tail_off,
                              int batch, cudaStream_t stream) {
    if (batch <= 0 || K <= 1) return BROLM_OK;
    if (C <= 0) return BROLM_ERR_BAD_SIZE;
    if ((C + 255) / 256 > 65535) return BROLM_ERR_TOO_LARGE;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid(batch, (C + 255) / 256);
    if (x_dtype == BROLM_F32)
        return launch_pdl(conv_tail_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, ldx, (const float*)in_bias, C, K,
                          s, tail_off);
    if (x_dtype == BROLM_BF16)
        return launch_pdl(conv_tail_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, ldx, (const float*)in_bias, C, K,
                          s, tail_off);
    return BROLM_ERR_BAD_DTYPE;
}

// out [tokens, width] = state * gelu_tanh(y_raw + yb) after the recurrence moved on; state at offset 0 of a slot's row.
BROLM_API int brolm_gated_scan(const void* pre, long ldpre, const void* u, long ldu, const void* y_raw, int y_dtype, long ldy,
                               const void* yb, const void* rb, const void* ib, const void* lam, float decay_scale, int width,
                               int bs, const void* cu_q, const void* kv_len, const void* slots, void* state, long state_stride,
                               void* out, int out_dtype, long ldo, int batch, cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    if (width <= 0 || bs <= 0 || width % bs) return BROLM_ERR_BAD_SIZE;
    if (batch > 65535) return BROLM_ERR_TOO_LARGE;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid((width + 127) / 128, batch);
#define BROLM_GS(Y, O) return launch_pdl(gated_scan_kernel<Y, O>, grid, dim3(128), 0, stream, (const float*)pre, ldpre,        \
        (const float*)u, ldu, (const Y*)y_raw, ldy, (const float*)yb, (const float*)rb, (const float*)ib, (const float*)lam, \
        decay_scale, width, bs, s, (O*)out, ldo)
    if (y_dtype == BROLM_F32 && out_dtype == BROLM_F32) BROLM_GS(float, float);
    if (y_dtype == BROLM_F32 && out_dtype == BROLM_BF16) BROLM_GS(float, bf16);
    if (y_dtype == BROLM_BF16 && out_dtype == BROLM_BF16) BROLM_GS(bf16, bf16);
#undef BROLM_GS
    return BROLM_ERR_BAD_DTYPE;
}

// y [tokens, heads * P] float; the state matrix sits at offset 0 of a slot's row as [heads][P][N].
BROLM_API int brolm_ssm_scan(const void* xbc, long ldx, const void* dt_raw, int dt_dtype, long lddt, const void* dt_bias,
                             const void* A_log, const void* Dv, int heads, int groups, int P, int N, const void* cu_q,
                             const void* kv_len, const void* slots, void* state, long state_stride, void* y, long ldy,
                             int batch, cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0) return BROLM_ERR_BAD_SIZE;
    if (N > 256 || batch > 65535 || heads > 65535) return BROLM_ERR_TOO_LARGE;
    // as few states per thread as fit
    int nsplit = 1;
    while (nsplit < 32 && (N + nsplit - 1) / nsplit > 8) nsplit <<= 1;
    const int per = (N + nsplit - 1) / nsplit;
    const int VT = 128 / nsplit;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid((P + VT - 1) / VT, heads, batch);
    const size_t smem = (size_t)(2 * SSM_TC * N + SSM_TC * VT + 2 * SSM_TC) * sizeof(float);
#define BROLM_SSM(X, NPT) return launch_pdl(ssm_scan_kernel<X, NPT>, grid, dim3(128), smem, stream, (const float*)xbc, ldx,   \
        (const X*)dt_raw, lddt, (const float*)dt_bias, (const float*)A_log, (const float*)Dv, heads, groups, P, N, nsplit, s, \
        (float*)y, ldy)
#define BROLM_SSM_N(X)                    \
    do {                                  \
        if (per <= 2) BROLM_SSM(X, 2);    \
        if (per <= 4) BROLM_SSM(X, 4);    \
        if (per <= 8) BROLM_SSM(X, 8);    \
        BROLM_SSM(X, 16);                 \
    } while (0)
    if (dt_dtype == BROLM_F32) BROLM_SSM_N(float);
    if (dt_dtype == BROLM_BF16) BROLM_SSM_N(bf16);
#undef BROLM_SSM_N
#undef BROLM_SSM
    return BROLM_ERR_BAD_DTYPE;
}
