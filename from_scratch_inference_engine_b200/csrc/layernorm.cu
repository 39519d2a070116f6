// Layer norm with a gain and no bias, in the two forms a decoder step needs, and the cast of
// the 32-bit residual stream to the storage type of the matrix products.
//
//   plain        y[r] = T( LN(src[s]) * gain )            s = rows ? rows[r] : r, src is 32-bit
//   accumulate   x[r] += LN(src[r]) * gain;  y[r] = T(x[r])   src is a sublayer's output (type T)
//
// LN(v) = (v - mean(v)) / sqrt(mean((v - mean(v))^2) + eps): the variance is the mean of the
// squared deviations, taken in a second pass over the row (kept in shared memory).  Statistics,
// the gain and the residual sum are 32-bit whatever T is.
#include "common.cuh"

namespace fsie {

template <typename S, typename T>
__global__ void add_layernorm_kernel(const S* __restrict__ src, const int* __restrict__ rows,
                                     const float* __restrict__ gain, float* __restrict__ x,
                                     T* __restrict__ y, int width, float eps) {
    extern __shared__ float row_cache[];
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    const S* in = src + s * width;
    float sum = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = to_float(in[c]);
        row_cache[c] = v;
        sum += v;
    }
    const float mean = block_sum(sum, scratch) / (float)width;
    float sq = 0.f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float d = row_cache[c] - mean;
        sq += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)width + eps);
    float* xr = x ? x + (size_t)r * width : nullptr;
    T* yr = y ? y + (size_t)r * width : nullptr;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float v = (row_cache[c] - mean) * inv * gain[c];
        if (xr) {
            v += xr[c];
            xr[c] = v;
        }
        if (yr) yr[c] = from_float<T>(v);
    }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ x, T* __restrict__ y, long long count) {
    grid_dependency_wait();
    grid_dependents_go();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x)
        y[i] = from_float<T>(x[i]);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// accumulate = 0: src is float [*, width] (read at `rows` if given), y gets the normed rows.
// accumulate = 1: src is of the storage type, x (float) += LN(src) * gain, y (optional) = T(x).
int fsie_add_layernorm(const void* src, const int* rows, const float* gain, float* x, void* y,
                       int num_rows, int width, float eps, int accumulate, int dtype,
                       cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (width <= 0 || (!accumulate && !y) || (accumulate && !x)) return ERR_BAD_ARGUMENT;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : 128);
    int code = 0;
#define FSIE_LN(S, T)                                                                           \
    do {                                                                                        \
        if (smem > 48 * 1024)                                                                   \
            cudaFuncSetAttribute(add_layernorm_kernel<S, T>,                                    \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
        code = launch_dependent(add_layernorm_kernel<S, T>, num_rows, threads, smem, stream,    \
                                (const S*)src, rows, gain, accumulate ? x : nullptr, (T*)y,      \
                                width, eps);                                                     \
    } while (0)
    if (dtype == DTYPE_F32) {
        FSIE_LN(float, float);
    } else if (accumulate) {
        FSIE_LN(bf16, bf16);
    } else {
        FSIE_LN(float, bf16);
    }
#undef FSIE_LN
    return code;
}

int fsie_cast_rows(const float* x, void* y, long long count, int dtype, cudaStream_t stream) {
    if (count <= 0) return 0;
    const int threads = 256;
    const long long wanted = (count + threads - 1) / threads;
    const unsigned blocks = (unsigned)(wanted > 4096 ? 4096 : wanted);
    if (dtype == DTYPE_F32)
        return launch_dependent(cast_rows_kernel<float>, blocks, threads, 0, stream, x, (float*)y, count);
    return launch_dependent(cast_rows_kernel<bf16>, blocks, threads, 0, stream, x, (bf16*)y, count);
}

}  // extern "C"
