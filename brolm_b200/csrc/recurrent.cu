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

// The same for up to CONV_KMAX taps with a thread taking a run of CONV_RUN packed tokens of one channel: the taps'
// inputs slide through registers (newest last, unused places weigh zero), so a token of the same sequence as the one
// before it costs one load instead of K.
constexpr int CONV_KMAX = 8, CONV_RUN = 8;

template <typename X>
__global__ void __launch_bounds__(256) causal_conv_run_kernel(const X* __restrict__ x, long ldx, const float* __restrict__ in_bias,
                                                              const float* __restrict__ w, const float* __restrict__ bias, int C,
                                                              int K, int act, const int32_t* __restrict__ tok_seq,
                                                              const int32_t* __restrict__ positions, SeqArgs s, long tail_off,
                                                              float* __restrict__ out, long ldo, int tokens) {
    pdl_trigger();
    const int t0 = blockIdx.x * CONV_RUN;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float wr[CONV_KMAX], win[CONV_KMAX];
#pragma unroll
    for (int jj = 0; jj < CONV_KMAX; ++jj) {
        const int j = jj - (CONV_KMAX - K);
        wr[jj] = j >= 0 ? w[(size_t)c * K + j] : 0.0f;
        win[jj] = 0.0f;
    }
    const float ib = in_bias ? in_bias[c] : 0.0f, bo = bias ? bias[c] : 0.0f;
    pdl_wait();
    int prev_b = -1, prev_pos = -2;
    for (int i = 0; i < CONV_RUN && t0 + i < tokens; ++i) {
        const int t = t0 + i;
        const int pos = positions[t];
        if (pos < 0) { prev_b = -1; continue; }
        const int b = tok_seq[t];
        if (b == prev_b && pos == prev_pos + 1) {
#pragma unroll
            for (int jj = 0; jj < CONV_KMAX - 1; ++jj) win[jj] = win[jj + 1];
            win[CONV_KMAX - 1] = to_float(x[(size_t)t * ldx + c]) + ib;
        } else {
            const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
            const int first = s.kv_len[b] - q_len;
            const float* tail = s.state + (size_t)s.slots[b] * s.state_stride + tail_off;
#pragma unroll
            for (int jj = 0; jj < CONV_KMAX; ++jj) {
                const int j = jj - (CONV_KMAX - K);
                float v = 0.0f;
                if (j >= 0) {
                    const int q = pos - (K - 1) + j;
                    v = q >= first ? to_float(x[(size_t)(q0 + q - first) * ldx + c]) + ib
                                   : tail[(size_t)(q - first + K - 1) * C + c];
                }
                win[jj] = v;
            }
        }
        prev_b = b;
        prev_pos = pos;
        float acc = bo;
#pragma unroll
        for (int jj = 0; jj < CONV_KMAX; ++jj) acc = fmaf(wr[jj], win[jj], acc);
        if (act == CONV_SILU) acc = acc / (1.0f + expf(-acc));
        out[(size_t)t * ldo + c] = acc;
    }
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
//
// Two kernels.  gate_prep (every token and channel on its own) overwrites pre with log a (in r's place) and the
// input sqrt(1 - a^2) i u (in i's place).  gated_scan runs the recurrence; a sequence's tokens are cut into NSEG
// runs that are scanned side by side from zero, joined in order (a run of tokens acts on the state before it as
// S -> exp(sum of its log a) S + its own end state), and scanned once more from their true beginnings for the
// results.  One token per sequence (decoding) is one run.
// ---------------------------------------------------------------------------
// split_halves: u (float) -> [u_hi; u_lo] as bfloat16 rows, u_hi = bf16(u), u_lo = bf16(u - u_hi): together 16 bits of
// u's mantissa.  With bfloat16 matrices the two products are exact in float, so W u_hi + W u_lo is the float product
// of W with u cut to 16 bits, on the tensor cores.
__global__ void __launch_bounds__(256) split_halves_kernel(const float* __restrict__ u, long ldu, bf16* __restrict__ out, long ldo,
                                                           int rows, int cols) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    const float v = u[(size_t)t * ldu + c];
    const bf16 hi = __float2bfloat16_rn(v);
    out[(size_t)t * ldo + c] = hi;
    out[(size_t)(rows + t) * ldo + c] = __float2bfloat16_rn(v - __bfloat162float(hi));
}

__global__ void __launch_bounds__(256) gate_prep_kernel(float* __restrict__ pre, const float* __restrict__ pre_lo, long ldpre,
                                                        const float* __restrict__ u, long ldu,
                                                        const float* __restrict__ rb, const float* __restrict__ ib,
                                                        const float* __restrict__ lam, float decay_scale, int width, int bs,
                                                        const int32_t* __restrict__ positions) {
    pdl_trigger();
    const int t = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (positions[t] < 0 || c >= width) return;
    const int blk = c / bs, o = c - blk * bs;
    const size_t pr = (size_t)t * ldpre + (size_t)blk * 2 * bs + o, pi = pr + bs;
    const float sp = -decay_scale * softplus_f(lam[c]);
    const float bias_r = rb[c], bias_i = ib[c];
    pdl_wait();
    float zr = pre[pr], zi = pre[pi];
    if (pre_lo) {                                   // the gates' sums came as two products (split_halves)
        zr += pre_lo[pr];
        zi += pre_lo[pi];
    }
    const float r = sigmoid_f(zr + bias_r), g = sigmoid_f(zi + bias_i);
    const float log_a = sp * r;
    pre[pr] = log_a;
    pre[pi] = sqrtf(-expm1f(2.0f * log_a)) * g * u[(size_t)t * ldu + c];
}

constexpr int GS_CH = 16;        // channels of a block (the lanes of half a warp: 64 contiguous bytes a row)

template <typename Y, typename O, int NSEG>
__global__ void __launch_bounds__(GS_CH * NSEG) gated_scan_kernel(const float* __restrict__ pre, long ldpre, const Y* __restrict__ y_raw,
                                                                  long ldy, const float* __restrict__ yb, int width, int bs,
                                                                  SeqArgs s, O* __restrict__ out, long ldo) {
    __shared__ float seg_sum[NSEG][GS_CH], seg_end[NSEG][GS_CH];
    // A prompt's scan runs long on few warps: it is launched in plain stream order and lets nothing in early; only the
    // short form for single tokens takes part in programmatic launch.
    if (NSEG == 1) pdl_trigger();
    const int b = blockIdx.y, cl = threadIdx.x, seg = threadIdx.y;
    const int c = blockIdx.x * GS_CH + cl;
    const int kv_len = s.kv_len[b];
    if (kv_len <= 0) return;
    const bool ok = c < width;
    const int cc = ok ? c : 0;
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int blk = cc / bs, o = cc - blk * bs;
    const size_t pr = (size_t)blk * 2 * bs + o, pi = pr + bs;
    const float bias_y = yb ? yb[cc] : 0.0f;
    float* st = s.state + (size_t)s.slots[b] * s.state_stride + cc;
    const int L = (q_len + NSEG - 1) / NSEG;
    const int t_lo = min(q_len, seg * L), t_hi = min(q_len, t_lo + L);
    pdl_wait();
    constexpr int U = 4;
    float S;
    if (NSEG > 1) {
        float loc = 0.0f, sum = 0.0f;
        for (int t0 = t_lo; t0 < t_hi; t0 += U) {
            float la[U], d[U];
#pragma unroll
            for (int k = 0; k < U; ++k)
                if (t0 + k < t_hi) {
                    const size_t row = (size_t)(q0 + t0 + k) * ldpre;
                    la[k] = pre[row + pr];
                    d[k] = pre[row + pi];
                }
#pragma unroll
            for (int k = 0; k < U; ++k)
                if (t0 + k < t_hi) {
                    loc = fmaf(expm1f(la[k]), loc, loc) + d[k];
                    sum += la[k];
                }
        }
        seg_sum[seg][cl] = sum;
        seg_end[seg][cl] = loc;
        __syncthreads();
        if (seg == 0) {
            float run = *st;
            for (int g = 0; g < NSEG; ++g) {
                const float begin = run;
                run = fmaf(expm1f(seg_sum[g][cl]), run, run) + seg_end[g][cl];
                seg_end[g][cl] = begin;                       // from here on: the state a run starts from
            }
            if (ok) *st = run;
        }
        __syncthreads();
        S = seg_end[seg][cl];
    } else {
        S = *st;
    }
    for (int t0 = t_lo; t0 < t_hi; t0 += U) {
        float la[U], d[U], vy[U];
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (t0 + k < t_hi) {
                const size_t row = (size_t)(q0 + t0 + k);
                la[k] = pre[row * ldpre + pr];
                d[k] = pre[row * ldpre + pi];
                vy[k] = to_float(y_raw[row * ldy + cc]);
            }
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (t0 + k < t_hi) {
                S = fmaf(expm1f(la[k]), S, S) + d[k];
                if (ok) out[(size_t)(q0 + t0 + k) * ldo + c] = from_float<O>(S * gelu_tanh_f(vy[k] + bias_y));
            }
    }
    if (NSEG == 1 && ok) *st = S;
}

// ---------------------------------------------------------------------------
// Selective state space.  Per head h (group g = h / (heads / groups)), S of N x P floats, kept as [h][p][n]:
//   dt = softplus(dt_raw[t][h] + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt * B[t][g] x[t][h]^T
//   y[t][h] = S^T C[t][g] + D[h] x[t][h]
// xbc row t: [ x: heads*P | B: groups*N | C: groups*N ] float (after the convolution and its activation).
// A block of 128 threads takes one (sequence, head) and 128 / nsplit tiles of PT values of p; thread (tile, s) keeps
// PT x NPT states in registers, n = jj * 4 nsplit + 4 s + e (jj < NPT / 4, e < 4), so that it reads B and C as
// float4, each for PT values of p at once, and the nsplit lanes of a tile read one contiguous run.  The sums over
// n of a tile's PT results are folded across the lanes by exchanging halves (five shuffles for four sums over
// sixteen lanes).  The tokens of a sequence are staged sixteen at a time through two buffers filled by cp.async,
// the next sixteen on their way while these are worked on; N is padded with zeros to nsplit * NPT in shared
// memory, so the inner loop has no bounds.
// ---------------------------------------------------------------------------
constexpr int SSM_TC = 16;

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16f(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <typename X, int NPT, int PT, int NS>       // NS: the lanes per tile when known at compile time, else 0
__global__ void __launch_bounds__(128) ssm_scan_kernel(const float* __restrict__ xbc, long ldx, const X* __restrict__ dt_raw, long lddt,
                                                       const float* __restrict__ dt_bias, const float* __restrict__ A_log,
                                                       const float* __restrict__ Dv, int heads, int groups, int P, int N,
                                                       int nsplit_rt, int vec, int early, SeqArgs s, float* __restrict__ y,
                                                       long ldy) {
    extern __shared__ __align__(16) float sm[];
    // A prompt's scan runs long on one or two warps a scheduler: it is launched in plain stream order (let in early, its
    // blocks land unevenly on the SMs and it takes 0.93 instead of 0.48 ms) and lets nothing in early; only a step of
    // single tokens takes part in programmatic launch.
    if (early) pdl_trigger();
    const int nsplit = NS > 0 ? NS : nsplit_rt;
    const int VP = (128 / nsplit) * PT, NP = nsplit * NPT;            // values of p a block takes; padded N
    const int stage_floats = 2 * SSM_TC * NP + SSM_TC * VP + SSM_TC;   // B, C, x, raw dt
    float* sdt = sm + 2 * stage_floats;     // [TC]
    float* sem1 = sdt + SSM_TC;             // [TC]  decay - 1
    const int b = blockIdx.z, h = blockIdx.y, g = h / (heads / groups);
    const int kv_len = s.kv_len[b];
    if (kv_len <= 0) return;
    const int q0 = s.cu_q[b], q_len = s.cu_q[b + 1] - q0;
    const int sl = threadIdx.x % nsplit, tile = threadIdx.x / nsplit;
    const int p0 = blockIdx.x * VP, pt0 = p0 + tile * PT;              // this thread's p: pt0 .. pt0 + PT - 1
    const float A = -expf(A_log[h]), D = Dv[h], dtb = dt_bias[h];
    float* st = s.state + (size_t)s.slots[b] * s.state_stride + (size_t)h * P * N;
    const int inner = heads * P;
    const size_t offB = (size_t)inner + (size_t)g * N, offC = (size_t)inner + (size_t)(groups + g) * N;
    for (int i = threadIdx.x; i < 2 * stage_floats + 2 * SSM_TC; i += 128) sm[i] = 0.0f;
    __syncthreads();
    pdl_wait();

    auto issue = [&](int chunk) {
        float* base = sm + (chunk & 1) * stage_floats;
        float* sB = base;
        float* sC = sB + SSM_TC * NP;
        float* sx = sC + SSM_TC * NP;
        float* sraw = sx + SSM_TC * VP;
        const int t0 = chunk * SSM_TC, n_tok = min(SSM_TC, q_len - t0);
        if (vec) {
            const int n4 = N >> 2;
            for (int idx = threadIdx.x; idx < n_tok * n4; idx += 128) {
                const int tt = idx / n4, n = (idx - tt * n4) << 2;
                const float* row = xbc + (size_t)(q0 + t0 + tt) * ldx;
                cp_async16f(sB + tt * NP + n, row + offB + n);
                cp_async16f(sC + tt * NP + n, row + offC + n);
            }
        } else {
            for (int idx = threadIdx.x; idx < n_tok * N; idx += 128) {
                const int tt = idx / N, n = idx - tt * N;
                const float* row = xbc + (size_t)(q0 + t0 + tt) * ldx;
                cp_async4(sB + tt * NP + n, row + offB + n);
                cp_async4(sC + tt * NP + n, row + offC + n);
            }
        }
        for (int idx = threadIdx.x; idx < n_tok * VP; idx += 128) {
            const int tt = idx / VP, v = idx - tt * VP;
            if (p0 + v < P) cp_async4(sx + tt * VP + v, xbc + (size_t)(q0 + t0 + tt) * ldx + (size_t)h * P + p0 + v);
        }
        if (threadIdx.x < n_tok) {
            const X* src = dt_raw + (size_t)(q0 + t0 + threadIdx.x) * lddt + h;
            if (sizeof(X) == 4) cp_async4(sraw + threadIdx.x, reinterpret_cast<const float*>(src));
            else sraw[threadIdx.x] = to_float(*src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float S[PT][NPT];
#pragma unroll
    for (int pi = 0; pi < PT; ++pi)
#pragma unroll
        for (int jj = 0; jj < NPT / 4; ++jj)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = jj * 4 * nsplit + 4 * sl + e;
                S[pi][4 * jj + e] = (pt0 + pi < P && n < N) ? st[(size_t)(pt0 + pi) * N + n] : 0.0f;
            }
    const int n_chunks = (q_len + SSM_TC - 1) / SSM_TC;
    issue(0);
    for (int k = 0; k < n_chunks; ++k) {
        if (k + 1 < n_chunks) {
            issue(k + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* base = sm + (k & 1) * stage_floats;
        const float* sx = base + 2 * SSM_TC * NP;
        const int t0 = k * SSM_TC, n_tok = min(SSM_TC, q_len - t0);
        if (threadIdx.x < n_tok) {
            const float dt = softplus_f(sx[SSM_TC * VP + threadIdx.x] + dtb);
            sdt[threadIdx.x] = dt;
            sem1[threadIdx.x] = expm1f(A * dt);            // decay - 1: the decay is applied as S + (decay - 1) S
        }
        __syncthreads();
#pragma unroll 4
        for (int tt = 0; tt < n_tok; ++tt) {
            const float dt = sdt[tt], em1 = sem1[tt];
            float xv[PT], dx[PT], acc[PT];
#pragma unroll
            for (int pi = 0; pi < PT; ++pi) {
                xv[pi] = sx[tt * VP + tile * PT + pi];
                dx[pi] = dt * xv[pi];
                acc[pi] = 0.0f;
            }
            const float4* rb = reinterpret_cast<const float4*>(base + tt * NP) + sl;
            const float4* rc = reinterpret_cast<const float4*>(base + SSM_TC * NP + tt * NP) + sl;
#pragma unroll
            for (int jj = 0; jj < NPT / 4; ++jj) {
                const float4 b4 = rb[jj * nsplit], c4 = rc[jj * nsplit];
                const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, cc[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int pi = 0; pi < PT; ++pi)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float v = fmaf(dx[pi], bb[e], fmaf(em1, S[pi][4 * jj + e], S[pi][4 * jj + e]));
                        S[pi][4 * jj + e] = v;
                        acc[pi] = fmaf(v, cc[e], acc[pi]);
                    }
            }
            float* yrow = y + (size_t)(q0 + t0 + tt) * ldy + (size_t)h * P;
            if (PT == 4 && nsplit >= 4) {
                // lanes fold their four sums by halves: after two exchanges lane (bit1, bit0) of a group of four holds the
                // group's sum for p = 2 bit0 + bit1; the groups of four are then added up
                const bool b0 = sl & 1, b1 = sl & 2;
                const float r0 = (b0 ? acc[2 % PT] : acc[0]) + __shfl_xor_sync(0xffffffffu, b0 ? acc[0] : acc[2 % PT], 1);
                const float r1 = (b0 ? acc[3 % PT] : acc[1 % PT]) + __shfl_xor_sync(0xffffffffu, b0 ? acc[1 % PT] : acc[3 % PT], 1);
                float v = (b1 ? r1 : r0) + __shfl_xor_sync(0xffffffffu, b1 ? r0 : r1, 2);
                for (int o = 4; o < nsplit; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                const int pi = 2 * (sl & 1) + ((sl >> 1) & 1);
                if (sl < 4 && pt0 + pi < P)
                    yrow[pt0 + pi] = fmaf(D, b0 ? (b1 ? xv[3 % PT] : xv[2 % PT]) : (b1 ? xv[1 % PT] : xv[0]), v);
            } else if (PT == 2 && nsplit >= 2) {
                const bool b0 = sl & 1;
                float v = (b0 ? acc[1 % PT] : acc[0]) + __shfl_xor_sync(0xffffffffu, b0 ? acc[0] : acc[1 % PT], 1);
                for (int o = 2; o < nsplit; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (sl < 2 && pt0 + sl < P) yrow[pt0 + sl] = fmaf(D, b0 ? xv[1 % PT] : xv[0], v);
            } else {
#pragma unroll
                for (int pi = 0; pi < PT; ++pi) {
                    float v = acc[pi];
                    for (int o = nsplit >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                    if (sl == 0 && pt0 + pi < P) yrow[pt0 + pi] = fmaf(D, xv[pi], v);
                }
            }
        }
        __syncthreads();                                   // the buffer is free for the chunk after next
    }
#pragma unroll
    for (int pi = 0; pi < PT; ++pi)
#pragma unroll
        for (int jj = 0; jj < NPT / 4; ++jj)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int n = jj * 4 * nsplit + 4 * sl + e;
                if (pt0 + pi < P && n < N) st[(size_t)(pt0 + pi) * N + n] = S[pi][4 * jj + e];
            }
}

// ---------------------------------------------------------------------------
// The gates' block-diagonal products for a handful of tokens (decoding), float throughout:
//   out[r][g * o_goff + n] = sum_k w[g][n][k] * a[r][g * a_goff + k],   r < rows <= R
// A block takes one group g and 32 outputs; its rows of a are staged in shared memory; a warp takes an output at a
// time, its lanes stride over k (one coalesced pass over the matrix row, used for every token), and adds the lanes'
// sums by one fixed tree, so a token's result does not depend on the others in the step.
// ---------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(256) block_matvec_kernel(const float* __restrict__ a, long lda, long a_goff,
                                                           const float* __restrict__ w, float* __restrict__ out, long ldo,
                                                           long o_goff, int rows, int N, int K) {
    extern __shared__ float sa[];                      // [rows][K]
    pdl_trigger();
    const int g = blockIdx.x, n0 = blockIdx.y * 32;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    pdl_wait();
    for (int idx = threadIdx.x; idx < rows * K; idx += 256) {
        const int r = idx / K, k = idx - r * K;
        sa[idx] = a[(size_t)r * lda + (size_t)g * a_goff + k];
    }
    __syncthreads();
    for (int n = n0 + warp; n < min(N, n0 + 32); n += 8) {
        const float* wr = w + ((size_t)g * N + n) * K;
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.0f;
        for (int k = lane; k < K; k += 32) {
            const float wv = wr[k];
#pragma unroll
            for (int r = 0; r < R; ++r)
                if (r < rows) acc[r] = fmaf(wv, sa[r * K + k], acc[r]);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float v = warp_sum(acc[r]);
            if (lane == 0 && r < rows) out[(size_t)r * ldo + (size_t)g * o_goff + n] = v;
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
    if (K <= CONV_KMAX && tokens > 64) {       // a prompt: runs of tokens per thread
        dim3 rgrid((tokens + CONV_RUN - 1) / CONV_RUN, (C + 255) / 256);
        if (x_dtype == BROLM_F32)
            return launch_pdl(causal_conv_run_kernel<float>, rgrid, dim3(256), 0, stream, (const float*)x, ldx,
                              (const float*)in_bias, (const float*)w, (const float*)bias, C, K, act, (const int32_t*)tok_seq,
                              (const int32_t*)positions, s, tail_off, (float*)out, ldo, tokens);
        if (x_dtype == BROLM_BF16)
            return launch_pdl(causal_conv_run_kernel<bf16>, rgrid, dim3(256), 0, stream, (const bf16*)x, ldx,
                              (const float*)in_bias, (const float*)w, (const float*)bias, C, K, act, (const int32_t*)tok_seq,
                              (const int32_t*)positions, s, tail_off, (float*)out, ldo, tokens);
        return BROLM_ERR_BAD_DTYPE;
    }
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
// pre is overwritten (log a and the recurrence's input take the places of the gates' sums).
BROLM_API int brolm_split_halves(const void* u, long ldu, void* out, long ldo, int rows, int cols, cudaStream_t stream) {
    if (rows <= 0 || cols <= 0) return BROLM_OK;
    if ((cols + 255) / 256 > 65535) return BROLM_ERR_TOO_LARGE;
    return launch_pdl(split_halves_kernel, dim3(rows, (cols + 255) / 256), dim3(256), 0, stream, (const float*)u, ldu, (bf16*)out,
                      ldo, rows, cols);
}

// pre_lo: null, or the second of two products whose sum is the gates' sums (same layout and row stride as pre).
BROLM_API int brolm_gated_scan(void* pre, const void* pre_lo, long ldpre, const void* u, long ldu, const void* y_raw, int y_dtype, long ldy,
                               const void* yb, const void* rb, const void* ib, const void* lam, float decay_scale, int width,
                               int bs, const void* positions, const void* cu_q, const void* kv_len, const void* slots,
                               void* state, long state_stride, void* out, int out_dtype, long ldo, int batch, int tokens,
                               int max_q_len, cudaStream_t stream) {
    if (batch <= 0 || tokens <= 0) return BROLM_OK;
    if (width <= 0 || bs <= 0 || width % bs) return BROLM_ERR_BAD_SIZE;
    if (batch > 65535 || (width + 255) / 256 > 65535) return BROLM_ERR_TOO_LARGE;
    int st = launch_pdl(gate_prep_kernel, dim3(tokens, (width + 255) / 256), dim3(256), 0, stream, (float*)pre,
                        (const float*)pre_lo, ldpre,
                        (const float*)u, ldu, (const float*)rb, (const float*)ib, (const float*)lam, decay_scale, width, bs,
                        (const int32_t*)positions);
    if (st) return st;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid((width + GS_CH - 1) / GS_CH, batch);
#define BROLM_GS(Y, O)                                                                                                          \
    do {                                                                                                                        \
        if (max_q_len > 32)                                                                                                     \
            return launch_in_order(gated_scan_kernel<Y, O, 32>, grid, dim3(GS_CH, 32), 0, stream, (const float*)pre, ldpre,       \
                              (const Y*)y_raw, ldy, (const float*)yb, width, bs, s, (O*)out, ldo);                              \
        return launch_pdl(gated_scan_kernel<Y, O, 1>, grid, dim3(GS_CH, 1), 0, stream, (const float*)pre, ldpre,                \
                          (const Y*)y_raw, ldy, (const float*)yb, width, bs, s, (O*)out, ldo);                                  \
    } while (0)
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
                             int batch, int max_q_len, cudaStream_t stream) {
    if (batch <= 0) return BROLM_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0) return BROLM_ERR_BAD_SIZE;
    if (N > 256 || batch > 65535 || heads > 65535) return BROLM_ERR_TOO_LARGE;
    // states per thread and value of p (a multiple of four, at most 16) and lanes per tile: the least padding of N,
    // then eight states (the balance of loads from shared memory against shuffles), then the fewest lanes
    static const int kinds[4] = {8, 16, 12, 4};
    int nsplit = 32, npt = 16, best = 1 << 30;
    for (int k = 0; k < 4; ++k)
        for (int ns = 1; ns <= 32; ns <<= 1) {
            const int padded = ns * kinds[k];
            if (padded >= N && padded < best) { best = padded; nsplit = ns; npt = kinds[k]; }
        }
    // values of p per thread: four, unless that leaves the device with less than one warp per scheduler (one long
    // sequence alone: the loop over its tokens is a chain of dependent steps that only more warps can fill)
    const int early = max_q_len <= 32 ? 1 : 0;
    int pt = 4;
    while (pt > 1 && (long long)batch * heads * ((P + pt - 1) / pt) * nsplit < 1LL * 4 * 32 * device_sm_count()) pt >>= 1;
    if (const char* e = getenv("BROLM_SSM_PT")) {          // (for measurements)
        const int want = atoi(e);
        if (want == 1 || want == 2 || want == 4) pt = want;
    }
    const int VP = (128 / nsplit) * pt;
    const int vec = N % 4 == 0 && ldx % 4 == 0 && (heads * P) % 4 == 0 && ((uintptr_t)xbc & 15) == 0;
    const SeqArgs s = seq_args(cu_q, kv_len, slots, state, state_stride);
    dim3 grid((P + VP - 1) / VP, heads, batch);
    const size_t smem = (size_t)(2 * (2 * SSM_TC * nsplit * npt + SSM_TC * VP + SSM_TC) + 2 * SSM_TC) * sizeof(float);
#define BROLM_SSM(NPT, PT, NS)                                                                                                 \
    do {                                                                                                                       \
        if (smem > 48 * 1024) {                                                                                                \
            cudaError_t e = cudaFuncSetAttribute(ssm_scan_kernel<float, NPT, PT, NS>,                                          \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
            if (e != cudaSuccess) return (int)e;                                                                               \
        }                                                                                                                      \
        if (!early)                                                                                                            \
            return launch_in_order(ssm_scan_kernel<float, NPT, PT, NS>, grid, dim3(128), smem, stream, (const float*)xbc, ldx, \
                                   (const float*)dt_raw, lddt, (const float*)dt_bias, (const float*)A_log, (const float*)Dv,   \
                                   heads, groups, P, N, nsplit, vec, early, s, (float*)y, ldy);                                \
        return launch_pdl(ssm_scan_kernel<float, NPT, PT, NS>, grid, dim3(128), smem, stream, (const float*)xbc, ldx,          \
                          (const float*)dt_raw, lddt, (const float*)dt_bias, (const float*)A_log, (const float*)Dv, heads,     \
                          groups, P, N, nsplit, vec, early, s, (float*)y, ldy);                                                \
    } while (0)
    // eight states per thread is what sizes of 64 states and more get: those know their lanes at compile time
#define BROLM_SSM_N(PT)                                   \
    do {                                                  \
        if (npt == 4) BROLM_SSM(4, PT, 0);                \
        if (npt == 8 && nsplit == 8) BROLM_SSM(8, PT, 8);   \
        if (npt == 8 && nsplit == 16) BROLM_SSM(8, PT, 16); \
        if (npt == 8 && nsplit == 32) BROLM_SSM(8, PT, 32); \
        if (npt == 8) BROLM_SSM(8, PT, 0);                \
        if (npt == 12) BROLM_SSM(12, PT, 0);              \
        BROLM_SSM(16, PT, 0);                             \
    } while (0)
    if (dt_dtype != BROLM_F32) return BROLM_ERR_BAD_DTYPE;
    if (pt == 4) BROLM_SSM_N(4);
    if (pt == 2) BROLM_SSM_N(2);
    BROLM_SSM_N(1);
#undef BROLM_SSM_N
#undef BROLM_SSM
}

// out[r][g * o_goff + n] = sum_k w[g][n][k] a[r][g * a_goff + k] for rows <= 16 and rows * K <= 12288, all float.
BROLM_API int brolm_block_matvec_f32(const void* a, long lda, long a_goff, const void* w, void* out, long ldo, long o_goff,
                                     int rows, int groups, int N, int K, cudaStream_t stream) {
    if (rows <= 0 || groups <= 0 || N <= 0) return BROLM_OK;
    if (K <= 0) return BROLM_ERR_BAD_SIZE;
    if (rows > 16 || (long long)rows * K > 12288 || (N + 31) / 32 > 65535) return BROLM_ERR_TOO_LARGE;
    dim3 grid(groups, (N + 31) / 32);
    const size_t smem = (size_t)rows * K * sizeof(float);
#define BROLM_BM(R) return launch_pdl(block_matvec_kernel<R>, grid, dim3(256), smem, stream, (const float*)a, lda, a_goff, \
                                      (const float*)w, (float*)out, ldo, o_goff, rows, N, K)
    if (rows <= 2) BROLM_BM(2);
    if (rows <= 4) BROLM_BM(4);
    if (rows <= 8) BROLM_BM(8);
    BROLM_BM(16);
#undef BROLM_BM
}
