// Latent attention, the row-wise step between the input projection and the
// attention kernel.  A token's projection row holds, head by head, the queries
// [unrotated (dn) | rotated (dr)] and then the compressed key/value row
// [a (R) | kr (dr)].  This kernel makes, per token:
//
//   the latent row   [ a / sqrt(mean(a^2) + eps) * g  |  rot(kr, pos)  |  0 .. ]   (width Dp >= R + dr)
//   written to the packed rows of the step and to the token's place in the paged cache, and
//   the rotated query parts  rot(qr_h, pos)  at columns R .. R + dr of head h of the
//   queries in latent space (width Dp per head; the first R columns come from the per-head
//   product with the keys' up-projection, the columns beyond R + dr are zero).
//
// With the queries in latent space the scores are plain dot products with the cached row,
// (q_n . W_uk c + q_r . k_r) = ((W_uk^T q_n) . c + q_r . k_r), and the cached row serves as the
// value as well (its first R columns, up-projected after the weighted sum).
//
// rot: pairs (i, i + rd/2), i < rd/2, of the first rd <= dr entries turn by pos * base^(-2i/rd)
// (cos and sin from a table built by the host); the entries beyond rd pass unchanged.
// The norm's statistics, the gain and the rotation are float; one rounding to the element type.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(128) latent_rows_kernel(
    const T* __restrict__ proj, long ld_proj, int q_cols,          // queries at 0, compressed row at q_cols
    const int32_t* __restrict__ positions, const float* __restrict__ cos_sin, int rd,
    const T* __restrict__ gain, float eps, int heads, int dn, int dr, int R, int Dp,
    T* __restrict__ lat, T* __restrict__ qlat, T* __restrict__ pages, const int32_t* __restrict__ cache_rows) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const T* row = proj + (size_t)t * ld_proj;
    const T* a = row + q_cols;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) {
        const float v = to_float(a[i]);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)R + eps);
    const int cr = cache_rows ? cache_rows[t] : -1;
    T* l0 = lat + (size_t)t * Dp;
    T* l1 = (pages && cr >= 0 && pos >= 0) ? pages + (size_t)cr * Dp : nullptr;
    const int half = rd >> 1;
    const float* cs = (pos >= 0 && cos_sin) ? cos_sin + (size_t)pos * half * 2 : nullptr;
    auto turned = [&](const T* v, int i) -> float {      // entry i of rot(v, pos)
        if (i >= rd || !cs) return to_float(v[i]);
        const int j = i < half ? i : i - half;
        const float c = cs[2 * j], s = cs[2 * j + 1];
        const float u = to_float(v[j]), w = to_float(v[j + half]);
        return i < half ? u * c - w * s : w * c + u * s;
    };
    for (int i = threadIdx.x; i < Dp; i += blockDim.x) {
        float v = 0.0f;
        if (i < R) v = to_float(a[i]) * inv * to_float(gain[i]);
        else if (i < R + dr) v = turned(a + R, i - R);
        const T o = from_float<T>(v);
        l0[i] = o;
        if (l1) l1[i] = o;
    }
    const int tail = Dp - R;                             // columns R .. Dp of every head of the latent queries
    for (int idx = threadIdx.x; idx < heads * tail; idx += blockDim.x) {
        const int h = idx / tail, i = idx - h * tail;
        const float v = i < dr ? turned(row + (size_t)h * (dn + dr) + dn, i) : 0.0f;
        qlat[((size_t)t * heads + h) * Dp + R + i] = from_float<T>(v);
    }
}

}  // namespace

BROLM_API int brolm_latent_rows(int dtype, const void* proj, long ld_proj, int q_cols, const void* positions,
                                const void* cos_sin, int rd, const void* gain, float eps, int heads, int dn, int dr,
                                int R, int Dp, void* lat, void* qlat, void* pages, const void* cache_rows, int tokens,
                                cudaStream_t stream) {
    if (tokens <= 0) return BROLM_OK;
    if (heads <= 0 || dn < 0 || dr < 0 || R <= 0 || Dp < R + dr || rd < 0 || rd > dr || (rd & 1))
        return BROLM_ERR_BAD_SIZE;
    if (dtype == BROLM_F32)
        latent_rows_kernel<float><<<tokens, 128, 0, stream>>>(
            (const float*)proj, ld_proj, q_cols, (const int32_t*)positions, (const float*)cos_sin, rd,
            (const float*)gain, eps, heads, dn, dr, R, Dp, (float*)lat, (float*)qlat, (float*)pages,
            (const int32_t*)cache_rows);
    else if (dtype == BROLM_BF16)
        latent_rows_kernel<bf16><<<tokens, 128, 0, stream>>>(
            (const bf16*)proj, ld_proj, q_cols, (const int32_t*)positions, (const float*)cos_sin, rd,
            (const bf16*)gain, eps, heads, dn, dr, R, Dp, (bf16*)lat, (bf16*)qlat, (bf16*)pages,
            (const int32_t*)cache_rows);
    else
        return BROLM_ERR_BAD_DTYPE;
    return launch_status();
}
