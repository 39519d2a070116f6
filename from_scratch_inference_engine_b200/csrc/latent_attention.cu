// The steps of attention over a latent cache that are neither a plain matrix product nor the
// attention itself.  Per token the cache keeps ONE row shared by all heads: a normed latent vector
// c (rank columns) and a rotated key part (rope columns).  A head's unrotated keys and its values
// are linear in c (k_h = U_h c, v_h = V_h c), so they are never formed: the query takes U_h over
// (q_h . U_h c = (U_h^T q_h) . c) and V_h is applied to the attention's output over c.
//
//   latent_prep    proj[t] = [ q: heads x (dim | rope) | lat: rank | kr: rope ]
//                  c  = lat / sqrt(mean(lat^2) + eps) * gain          -> cache row columns [0, rank)
//                  kr rotated (pairs 2i, 2i + 1 of the leading rotary_dim) -> columns [rank, rank + rope)
//                  each head's rope part of q, rotated the same way     -> qa[t, h, rank ...]
//   head_product   out[t, h, :] = W[h] x[t, h, :]   for W [heads, n, k]: U_h^T before the attention
//                  (x = the unrotated part of q, out = qa[t, h, 0 .. rank)), V_h after it.
//
// Norm statistics, angles and the products' sums are 32-bit; storage type T for proj, cache and qa.
#include "common.cuh"
#include <math.h>

namespace fsie {

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                   const float* __restrict__ cos_sin, int table_len,
                                   const int* __restrict__ slot_of, T* __restrict__ pages,
                                   long long page_stride, int page_size, const float* __restrict__ gain,
                                   float eps, T* __restrict__ qa, int heads, int dim, int rope, int rank,
                                   int rotary_dim, int* __restrict__ error) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependents_go();
    const int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;       // cos of pair i at [i], sin at [half + i]
    const T* row = proj + (size_t)t * ld;
    const int qd = dim + rope, row_width = rank + rope;
    // queries: the rope part of every head, rotated, behind the rank columns the product will fill
    for (int e = threadIdx.x; e < heads * rope; e += blockDim.x) {
        const int h = e / rope, d = e - h * rope;
        const T* src = row + h * qd + dim;
        float val = to_float(src[d]);
        if (d < rotary_dim) {
            const int i = d >> 1;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(src[d ^ 1]);
            val = (d & 1) ? val * c + other * s : val * c - other * s;
        }
        qa[((size_t)t * heads + h) * row_width + rank + d] = from_float<T>(val);
    }
    const int slot = slot_of ? slot_of[t] : -1;
    const T* lat = row + heads * qd;
    float ss = 0.f;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) {
        const float v = to_float(lat[d]);
        ss += v * v;
    }
    ss = block_sum(ss, scratch);
    if (slot < 0) return;
    const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
    T* dst = pages + (long long)(slot / page_size) * page_stride + (long long)(slot % page_size) * row_width;
    for (int d = threadIdx.x; d < rank; d += blockDim.x)
        dst[d] = from_float<T>((to_float(lat[d]) * scale) * gain[d]);
    const T* kr = lat + rank;
    for (int d = threadIdx.x; d < rope; d += blockDim.x) {
        float val = to_float(kr[d]);
        if (d < rotary_dim) {
            const int i = d >> 1;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(kr[d ^ 1]);
            val = (d & 1) ? val * c + other * s : val * c - other * s;
        }
        dst[rank + d] = from_float<T>(val);
    }
}

// out[t, h, n] = sum_k x[t, h, k] w[h, n, k]; a block owns 64 tokens x 64 outputs of one head,
// a thread 4 x 4 of them; k in steps of 16 through shared memory.
constexpr int HP_TILE = 64, HP_K = 16;

template <typename T>
__global__ void __launch_bounds__(256) head_product_kernel(const T* __restrict__ x, long long x_ld, int x_head,
                                                           const T* __restrict__ w, T* __restrict__ out,
                                                           long long out_ld, int out_head, int tokens,
                                                           int n, int k) {
    __shared__ float xs[HP_K][HP_TILE + 4];
    __shared__ float ws[HP_K][HP_TILE + 4];
    const int h = blockIdx.z, t0 = blockIdx.x * HP_TILE, n0 = blockIdx.y * HP_TILE;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    grid_dependency_wait();
    grid_dependents_go();
    const T* xh = x + (size_t)h * x_head;
    const T* wh = w + (size_t)h * n * k;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < k; k0 += HP_K) {
        for (int e = threadIdx.x; e < HP_TILE * HP_K; e += 256) {
            const int r = e / HP_K, kk = e - r * HP_K;
            const int t = t0 + r, c = n0 + r, kc = k0 + kk;
            xs[kk][r] = (t < tokens && kc < k) ? to_float(xh[(size_t)t * x_ld + kc]) : 0.f;
            ws[kk][r] = (c < n && kc < k) ? to_float(wh[(size_t)c * k + kc]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HP_K; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[kk][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx * 4 + j;
            if (c < n) out[(size_t)t * out_ld + (size_t)h * out_head + c] = from_float<T>(acc[i][j]);
        }
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// proj [tokens, ld]; pages: the cache entry's rows of rank + rope columns, `page_size` per page;
// qa [tokens, heads, rank + rope]; gain float32 [rank]; cos_sin [table_len, rotary_dim].
int fsie_latent_prep(const void* proj, int ld, const int* positions, const float* cos_sin, int table_len,
                     const int* slot_of, void* pages, long long page_stride, int page_size,
                     const float* gain, float eps, void* qa, int tokens, int heads, int dim, int rope,
                     int rank, int rotary_dim, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (heads <= 0 || dim < 0 || rope < 0 || rank <= 0 || rotary_dim < 0 || rotary_dim > rope ||
        (rotary_dim & 1) || ld < heads * (dim + rope) + rank + rope)
        return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return launch_dependent(latent_prep_kernel<float>, dim3(tokens), dim3(256), 0, stream,
                                (const float*)proj, ld, positions, cos_sin, table_len, slot_of, (float*)pages,
                                page_stride, page_size, gain, eps, (float*)qa, heads, dim, rope, rank,
                                rotary_dim, error);
    return launch_dependent(latent_prep_kernel<bf16>, dim3(tokens), dim3(256), 0, stream,
                            (const bf16*)proj, ld, positions, cos_sin, table_len, slot_of, (bf16*)pages,
                            page_stride, page_size, gain, eps, (bf16*)qa, heads, dim, rope, rank,
                            rotary_dim, error);
}

// x: head h of token t at t * x_ld + h * x_head (k columns); w [heads, n, k]; out: head h of token t
// at t * out_ld + h * out_head (n columns).
int fsie_head_product(const void* x, long long x_ld, int x_head, const void* w, void* out, long long out_ld,
                      int out_head, int tokens, int heads, int n, int k, int dtype, cudaStream_t stream) {
    if (tokens <= 0 || n <= 0) return 0;
    if (heads <= 0 || k <= 0 || heads > 65535) return ERR_BAD_ARGUMENT;
    const dim3 grid((tokens + HP_TILE - 1) / HP_TILE, (n + HP_TILE - 1) / HP_TILE, heads);
    if (grid.y > 65535) return ERR_UNSUPPORTED;
    if (dtype == DTYPE_F32)
        return launch_dependent(head_product_kernel<float>, grid, dim3(256), 0, stream, (const float*)x, x_ld,
                                x_head, (const float*)w, (float*)out, out_ld, out_head, tokens, n, k);
    return launch_dependent(head_product_kernel<bf16>, grid, dim3(256), 0, stream, (const bf16*)x, x_ld,
                            x_head, (const bf16*)w, (bf16*)out, out_ld, out_head, tokens, n, k);
}

}  // extern "C"
