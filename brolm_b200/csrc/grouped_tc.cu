// Routed experts with many rows per expert, on the 5th-generation tensor cores:
//     Y[row, :] = W[e] * A[row, :]     for the rows of expert e (W[e] stored (N, K), bfloat16, float accumulation)
// over the rows that the grouping kernel sorted by expert.  The structure is that of gemm_tc.cu (one persistent
// block of 192 threads per SM; a loader thread that issues TMA loads with the 128-byte swizzle into a ring of
// four stages; one thread that issues tcgen05.mma, M 128, N 256, into one of two accumulators in tensor
// memory; four warps that read a finished accumulator with tcgen05.ld while the next tile is multiplied into
// the other), with what a grouped product needs on top of it:
//   - the work list is made on the device: 128-row tiles (expert, first row), expert -1 past the last one,
//     times the 256-column tiles of N.  Every role walks the same list and stops at the first -1;
//   - A is one matrix of all rows in expert order, so a tile's rows are a plain box of it that may start at any
//     row; rows past the expert's last belong to the next expert (or are zeros past the end) and are computed
//     and dropped.  W is one matrix of experts * N rows; a box that runs past an expert's N rows likewise;
//   - the epilogue knows its row: first product  u[row] = act(gate[pair] * sum)  in bfloat16, second product
//     out[choice][token] = sum  in float, the pair being perm[row].
// For the first product the tokens' rows are first copied into expert order (gather_rows_kernel): a TMA box
// cannot follow a list of rows.
//
// Every wait on an mbarrier is bounded as in gemm_tc.cu; a wait that runs out ends the kernel early and
// brolm_grouped_tc_status() reports its code.
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;      // two accumulators of 256 columns

enum : int { ACT_NONE = 0, ACT_RELU2 = 1 };

__device__ int g_grouped_tc_error;      // 0, or the code of the first wait that ran out

struct GroupedTcArgs {
    void* out;
    long ldo;
    int out_f32, act, down;
    int N, K;
    int n_tiles, max_row_tiles;
    const int32_t* tile_group;
    const int32_t* tile_row0;
    const int32_t* offsets;
    const int32_t* perm;
    const float* scale;
    int top, tokens;
};

using namespace tc;

__device__ __forceinline__ bool wait_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_grouped_tc_error, code);
}
__device__ __forceinline__ bool drain_on(uint32_t bar, uint32_t parity, volatile int* give_up, int code) {
    return mbar_wait(bar, parity, give_up, &g_grouped_tc_error, code, true);
}
__device__ __forceinline__ float act_of(float v, int act) {
    if (act == ACT_RELU2) {
        v = fmaxf(v, 0.0f);
        return v * v;
    }
    return v;
}

// xs[s, :] = x[perm[s] / top, :]: the tokens' rows in expert order.  K a multiple of 8, rows 16-byte aligned.
__global__ void __launch_bounds__(256) gather_rows_kernel(const bf16* __restrict__ x, long ldx,
                                                          const int32_t* __restrict__ perm, int top, int pairs, int K,
                                                          bf16* __restrict__ xs) {
    const int chunks = K >> 3;
    for (int s = blockIdx.x; s < pairs; s += gridDim.x) {
        const int tok = perm[s] / top;
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)tok * ldx);
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)s * K);
        for (int c = threadIdx.x; c < chunks; c += blockDim.x) dst[c] = src[c];
    }
}

__global__ void __launch_bounds__(THREADS, 1) grouped_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                const __grid_constant__ CUtensorMap map_w,
                                                                GroupedTcArgs g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + STAGES * STAGE_BYTES);
    // barriers: full[STAGES], empty[STAGES], acc_full[2], acc_empty[2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* give_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t stage0 = smem_u32(base);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, acc_full0 = empty0 + 8 * STAGES,
                   acc_empty0 = acc_full0 + 16;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_kb = (g.K + BK - 1) / BK;
    const int total = g.max_row_tiles * g.n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(acc_full0 + 8 * s, 1);
            mbar_init(acc_empty0 + 8 * s, 4);     // one arrival per epilogue warp
        }
        give_up[0] = 0;
        give_up[1] = 0;
        give_up[2] = tc::g_stall_code;
        mbar_init_fence();
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
                const int rt = t / g.n_tiles, nt = t - rt * g.n_tiles;
                const int group = g.tile_group[rt];
                if (group < 0) break;
                const int row0 = g.tile_row0[rt];
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!wait_on(empty0 + 8 * s, ((it / STAGES) & 1) ^ 1, give_up, 1)) { ok = false; break; }
                    const uint32_t full = full0 + 8 * s, a_dst = stage0 + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full, STAGE_BYTES);
                    tma_load_2d(a_dst, &map_a, kb * BK, row0, full);
                    tma_load_2d(b_dst, &map_w, kb * BK, group * g.N + nt * BN, full);
                }
            }
            if (*give_up) {
                for (int j = max(0, it - STAGES); j < it; ++j)
                    drain_on(full0 + 8 * (j % STAGES), (j / STAGES) & 1, give_up, 4);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16(BM, BN);
            int it = 0, local = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++local) {
                if (g.tile_group[t / g.n_tiles] < 0) break;
                const int as = local & 1;
                ok = wait_on(acc_empty0 + 8 * as, ((local >> 1) & 1) ^ 1, give_up, 5);
                if (!ok) break;
                fence_after_sync();
                const uint32_t acc = tmem + as * BN;
                for (int kb = 0; kb < num_kb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = wait_on(full0 + 8 * s, (it / STAGES) & 1, give_up, 2);
                    if (!ok) break;
                    fence_after_sync();
                    const uint64_t a = desc_kmajor(stage0 + s * STAGE_BYTES), b = desc_kmajor(stage0 + s * STAGE_BYTES + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) umma(acc, a + 2 * k, b + 2 * k, idesc, (kb | k) != 0);
                    umma_commit(empty0 + 8 * s);
                }
                if (ok) umma_commit(acc_full0 + 8 * as);
            }
        }
    } else {
        const int quarter = warp & 3;                        // the 32 lanes of tensor memory this warp may read
        int local = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x, ++local) {
            const int rt = t / g.n_tiles, nt = t - rt * g.n_tiles;
            const int group = g.tile_group[rt];
            if (group < 0) break;
            const int row = g.tile_row0[rt] + quarter * 32 + lane;
            const bool valid = row < g.offsets[group + 1];
            float gate = 1.0f;
            long o_off = 0;
            if (valid) {
                const int p = g.perm[row];
                if (g.down) {
                    const int tok = p / g.top, choice = p - tok * g.top;
                    o_off = ((long)choice * g.tokens + tok) * g.ldo;
                } else {
                    gate = g.scale ? g.scale[p] : 1.0f;
                    o_off = (long)row * g.ldo;
                }
            }
            const int as = local & 1;
            const bool ready = wait_on(acc_full0 + 8 * as, (local >> 1) & 1, give_up, 3);
            if (!__all_sync(0xffffffffu, ready)) break;       // the warp leaves together
            fence_after_sync();
            const uint32_t acc = tmem + as * BN + ((uint32_t)(quarter * 32) << 16);
            const int col0 = nt * BN;
            for (int c = 0; c < BN; c += 32) {
                uint32_t v[32];
                __syncwarp();                                 // (rows that are dropped skipped the stores)
                tmem_ld32(acc + c, v);
                tmem_wait_ld();
                if (c + 32 >= BN) {
                    // everything of this accumulator is in registers: hand it back before the stores
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty0 + 8 * as);
                }
                const int col = col0 + c;
                if (!valid || col >= g.N) continue;
                float o[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = act_of(__uint_as_float(v[i]) * gate, g.act);
                const bool whole = col + 32 <= g.N;
                if (g.out_f32) {
                    float* dst = reinterpret_cast<float*>(g.out) + o_off + col;
                    if (whole && (g.ldo & 3) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                    } else {
                        for (int i = 0; i < 32; ++i) if (col + i < g.N) dst[i] = o[i];
                    }
                } else {
                    bf16* dst = reinterpret_cast<bf16*>(g.out) + o_off + col;
                    if (whole && (g.ldo & 7) == 0) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 q;
                            __nv_bfloat162* q2 = reinterpret_cast<__nv_bfloat162*>(&q);
#pragma unroll
                            for (int e = 0; e < 4; ++e) q2[e] = __floats2bfloat162_rn(o[i + 2 * e], o[i + 2 * e + 1]);
                            *reinterpret_cast<uint4*>(dst + i) = q;
                        }
                    } else {
                        for (int i = 0; i < 32; ++i) if (col + i < g.N) dst[i] = __float2bfloat16_rn(o[i]);
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TMEM_COLS);
}

constexpr size_t SMEM_BYTES = 1024 + (size_t)STAGES * STAGE_BYTES + (2 * STAGES + 4) * 8 + 16;

}  // namespace

// The tokens' rows in expert order: xs[s, :] = x[perm[s] / top, :], bfloat16, K a multiple of 8.
BROLM_API int brolm_gather_rows(const void* x, long ldx, const void* perm, int top, int pairs, int K, void* xs,
                                cudaStream_t stream) {
    if (pairs <= 0) return BROLM_OK;
    if (K <= 0 || K % 8 != 0 || ldx % 8 != 0 || top <= 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)x & 15) || ((uintptr_t)xs & 15)) return BROLM_ERR_ALIGNMENT;
    const int blocks = pairs < 148 * 16 ? pairs : 148 * 16;
    gather_rows_kernel<<<blocks, K >= 2048 ? 256 : 128, 0, stream>>>((const bf16*)x, ldx, (const int32_t*)perm, top, pairs, K,
                                                                    (bf16*)xs);
    return launch_status();
}

// One of the two products of routed experts over rows in expert order.  a (rows, K) with lda between rows; w
// (experts, N, K) contiguous; the tile list is one of 128-row tiles with room for max_row_tiles entries.
// down == 0: out (rows, N) in the operands' type or float, out[row] = act(scale[perm[row]] * (W[e] a[row]));
// down != 0: out float [top, tokens, N], a row's result at [choice, token] of its pair.
BROLM_API int brolm_experts_linear_tc(int down, const void* a, long lda, long rows, const void* w, int experts, void* out,
                                      long ldo, int out_f32, int act, int N, int K, const void* tile_group,
                                      const void* tile_row0, const void* offsets, const void* perm, const void* scale,
                                      int top, int tokens, int max_row_tiles, cudaStream_t stream) {
    if (rows <= 0 || max_row_tiles <= 0 || N <= 0) return BROLM_OK;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0) return BROLM_ERR_ALIGNMENT;
    if (((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15)) return BROLM_ERR_ALIGNMENT;
    if (act != ACT_NONE && act != ACT_RELU2) return BROLM_ERR_BAD_SIZE;
    CUtensorMap ma, mw;
    int st = make_map_2d(&ma, a, rows, K, lda, BM);
    if (st) return st;
    st = make_map_2d(&mw, w, (long long)experts * N, K, K, BN);
    if (st) return st;
    GroupedTcArgs g;
    g.out = out; g.ldo = ldo; g.out_f32 = out_f32; g.act = act; g.down = down; g.N = N; g.K = K;
    g.n_tiles = (N + BN - 1) / BN;
    g.max_row_tiles = max_row_tiles;
    g.tile_group = (const int32_t*)tile_group; g.tile_row0 = (const int32_t*)tile_row0;
    g.offsets = (const int32_t*)offsets; g.perm = (const int32_t*)perm; g.scale = (const float*)scale;
    g.top = top; g.tokens = tokens;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(grouped_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        raised = true;
    }
    const long long total = (long long)max_row_tiles * g.n_tiles;
    const int sms = device_sms();
    grouped_tc_kernel<<<(int)(total < sms ? total : sms), THREADS, SMEM_BYTES, stream>>>(ma, mw, g);
    return launch_status();
}

// 0 when no bounded wait of any launch so far ran out; else the code of the first one (1 loader, 2 and 5
// issuer, 3 epilogue, 4 drain).  Synchronises the device.  `reset` clears it.
BROLM_API int brolm_grouped_tc_status(int reset) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_grouped_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && v) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_grouped_tc_error, &zero, sizeof(int));
    }
    return v;
}

BROLM_WAIT_CONTROL(grouped_tc)
