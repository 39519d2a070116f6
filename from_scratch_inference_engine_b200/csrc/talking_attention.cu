// Attention whose softmax weights are mixed across heads ("talking heads"), over a sliding
// window that also keeps the first tokens of the sequence, fed by projections that pass a
// short causal convolution, whole-projection RMS norms and an interleaved rotation.
//
//   prepare   u = conv(projected q | k | v)              y_t = sum_j w[:, j] u_{t - taps + 1 + j}
//             q = rot(rms(u_q) * w_q)   k = rot(rms(u_k) * w_k)     rms over the WHOLE projection
//             v_head = u_v,head / sqrt(mean(u_v,head^2) + eps)
//             q -> a 32-bit buffer; k, v -> the pages of the cache
//   tails     the last taps - 1 projected rows of every request -> its state slot
//   attend    (talking_attention.cuh)  s_h(i, j) = (q_h,i . k_g(h),j) * scale  for visible j:
//                 j <= i and (window == 0 or i - j < window or j < keep_first)
//             p_h = softmax_j s_h          p'_h = sum_h' talk[h, h'] p_h'
//             o_h,i = sum_j p'_h(i, j) v_g(h),j
//
// Positions, norms, scores, softmax and the mixed weights are 32-bit whatever the storage type
// T of the projections and the pages.  Page layout: keys [kv_head][slot][dim] at k_pages +
// page * page_stride, values [kv_head][slot][vdim] at v_pages + page * page_stride.
#include "common.cuh"

namespace fsie {

// index of the request that token t belongs to: item_qstart is ascending, requests are packed
__device__ __forceinline__ int item_of_token(const int* __restrict__ item_qstart, int items, int t) {
    int lo = 0, hi = items - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (item_qstart[mid] <= t) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// ------------------------------------------------------------------------------ prepare
// One block per token.  `proj` [tokens, ld] holds q (wq columns), then k (wk), then v (wv);
// wk = wv = 0 for a layer that reads another layer's keys.  `tails` [slots, taps - 1, wq + wk +
// wv] holds the projected rows of the taps - 1 positions before the step's first token.
template <typename T>
__global__ void conv_norm_rotate_kernel(const T* __restrict__ proj, int ld, int items,
                                        const int* __restrict__ item_qstart,
                                        const int* __restrict__ item_pos0,
                                        const int* __restrict__ item_slots,
                                        const float* __restrict__ tails,
                                        const float* __restrict__ conv_w, int taps,
                                        const float* __restrict__ q_gain,
                                        const float* __restrict__ k_gain,
                                        const float* __restrict__ cos_sin, int table_len, int rot_dims,
                                        const int* __restrict__ slot_of, T* __restrict__ k_pages,
                                        T* __restrict__ v_pages, long long page_stride, int page_size,
                                        float* __restrict__ q_out, int heads, int kv_heads, int dim,
                                        int vdim, int has_kv, float eps, int* error) {
    extern __shared__ float y[];                       // the convolved row, then per-head value scales
    __shared__ float scratch[32];
    grid_dependency_wait();
    grid_dependents_go();
    const int t = blockIdx.x;
    const int item = item_of_token(item_qstart, items, t);
    const int slot = item_slots[item];
    if (slot < 0) return;                               // a padding entry of a fixed-size batch
    const int start = item_qstart[item], pos0 = item_pos0[item];
    const int pos = pos0 + (t - start);
    const int wq = heads * dim, wk = has_kv ? kv_heads * dim : 0, wv = has_kv ? kv_heads * vdim : 0;
    const int width = wq + wk + wv;
    const float* tail = tails ? tails + (size_t)slot * (taps - 1) * width : nullptr;
    float* v_scale = y + width;

    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int p = pos - taps + 1 + j;
            if (p < 0) continue;
            float u;
            if (p >= pos0) u = to_float(proj[(size_t)(start + p - pos0) * ld + c]);
            else u = tail[(size_t)(p - pos0 + taps - 1) * width + c];
            acc += conv_w[(size_t)c * taps + j] * u;
        }
        y[c] = acc;
    }
    __syncthreads();
    float sq = 0.f;
    for (int c = threadIdx.x; c < wq; c += blockDim.x) sq += y[c] * y[c];
    const float q_inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)wq + eps);
    float k_inv = 0.f;
    if (has_kv) {
        sq = 0.f;
        for (int c = threadIdx.x; c < wk; c += blockDim.x) sq += y[wq + c] * y[wq + c];
        k_inv = 1.0f / sqrtf(block_sum(sq, scratch) / (float)wk + eps);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
        for (int g = warp; g < kv_heads; g += warps) {
            const float* head = y + wq + wk + g * vdim;
            float s = 0.f;
            for (int c = lane; c < vdim; c += 32) s += head[c] * head[c];
            s = warp_sum(s);
            if (lane == 0) v_scale[g] = 1.0f / sqrtf(s / (float)vdim + eps);
        }
    }
    __syncthreads();

    int table_pos = pos;
    if (rot_dims > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        table_pos = 0;
    }
    const int half = rot_dims / 2;
    const float* cs = cos_sin + (size_t)table_pos * rot_dims;      // [cos (half) | sin (half)]
    const int slot_kv = has_kv ? slot_of[t] : -1;
    const long long page = slot_kv >= 0 ? slot_kv / page_size : 0;
    const int offset = slot_kv >= 0 ? slot_kv - (int)page * page_size : 0;

    // q and k: normed with their gains, pairs (2i, 2i + 1) of the first rot_dims of a head turned
    for (int c = threadIdx.x; c < wq + wk; c += blockDim.x) {
        const bool is_q = c < wq;
        const int local = is_q ? c : c - wq;
        const int h = local / dim, d = local - h * dim;
        const float inv = is_q ? q_inv : k_inv;
        const float* gain = is_q ? q_gain : k_gain;
        float value = y[c] * inv * gain[local];
        if (d < rot_dims) {
            const int partner = (d & 1) ? c - 1 : c + 1;
            const int plocal = (d & 1) ? local - 1 : local + 1;
            const float other = y[partner] * inv * gain[plocal];
            const float co = cs[d >> 1], si = cs[half + (d >> 1)];
            value = (d & 1) ? value * co + other * si : value * co - other * si;
        }
        if (is_q) {
            q_out[(size_t)t * wq + c] = value;
        } else if (slot_kv >= 0) {
            k_pages[page * page_stride + ((size_t)h * page_size + offset) * dim + d] = from_float<T>(value);
        }
    }
    if (slot_kv >= 0) {
        for (int c = threadIdx.x; c < wv; c += blockDim.x) {
            const int g = c / vdim, d = c - g * vdim;
            v_pages[page * page_stride + ((size_t)g * page_size + offset) * vdim + d] =
                from_float<T>(y[wq + wk + c] * v_scale[g]);
        }
    }
}

// ------------------------------------------------------------------------------- tails
// One block per request: row r of its new tail is the projected row of position
// end - (taps - 1) + r, which is a row of this step or, when the step brought fewer than
// taps - 1 tokens, row r + count of the old tail (read before anything overwrites it: a thread
// owns a channel and moves upwards).
template <typename T>
__global__ void conv_tails_kernel(const T* __restrict__ proj, int ld, const int* __restrict__ item_qstart,
                                  const int* __restrict__ item_qlen, const int* __restrict__ item_slots,
                                  float* __restrict__ tails, int taps, int width) {
    grid_dependency_wait();
    grid_dependents_go();
    const int item = blockIdx.x;
    const int slot = item_slots[item];
    if (slot < 0) return;
    const int start = item_qstart[item], count = item_qlen[item], keep = taps - 1;
    float* tail = tails + (size_t)slot * keep * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        for (int r = 0; r < keep; ++r) {
            const int back = keep - r;                  // how far before the end this row lies
            float u;
            if (back <= count) u = to_float(proj[(size_t)(start + count - back) * ld + c]);
            else u = tail[(size_t)(r + count) * width + c];
            tail[(size_t)r * width + c] = u;
        }
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_conv_norm_rotate(const void* proj, int ld, int tokens, int items, const int* item_qstart,
                          const int* item_pos0, const int* item_slots, const float* tails,
                          const float* conv_w, int taps, const float* q_gain, const float* k_gain,
                          const float* cos_sin, int table_len, int rot_dims, const int* slot_of,
                          void* k_pages, void* v_pages, long long page_stride, int page_size,
                          float* q_out, int heads, int kv_heads, int dim, int vdim, int has_kv,
                          float eps, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (items <= 0 || taps <= 0 || (taps > 1 && !tails) || rot_dims < 0 || rot_dims > dim || (rot_dims & 1))
        return ERR_BAD_ARGUMENT;
    const int width = heads * dim + (has_kv ? kv_heads * (dim + vdim) : 0);
    const size_t smem = (size_t)(width + kv_heads) * sizeof(float);
    if (smem > 200 * 1024) return ERR_UNSUPPORTED;
    const int threads = width >= 1024 ? 512 : 256;
    int code = 0;
#define FSIE_PREPARE(T)                                                                          \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(conv_norm_rotate_kernel<T>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        code = launch_dependent(conv_norm_rotate_kernel<T>, tokens, threads, smem, stream,       \
            (const T*)proj, ld, items, item_qstart, item_pos0, item_slots, tails, conv_w, taps,  \
            q_gain, k_gain, cos_sin, table_len, rot_dims, slot_of, (T*)k_pages, (T*)v_pages,     \
            page_stride, page_size, q_out, heads, kv_heads, dim, vdim, has_kv, eps, error);      \
    } while (0)
    if (dtype == DTYPE_F32) FSIE_PREPARE(float);
    else FSIE_PREPARE(bf16);
#undef FSIE_PREPARE
    return code;
}

int fsie_conv_tails(const void* proj, int ld, const int* item_qstart, const int* item_qlen,
                    const int* item_slots, int items, float* tails, int taps, int width, int dtype,
                    cudaStream_t stream) {
    if (items <= 0 || taps <= 1) return 0;
    if (dtype == DTYPE_F32)
        return launch_dependent(conv_tails_kernel<float>, items, 256, 0, stream, (const float*)proj, ld,
                                item_qstart, item_qlen, item_slots, tails, taps, width);
    return launch_dependent(conv_tails_kernel<bf16>, items, 256, 0, stream, (const bf16*)proj, ld,
                            item_qstart, item_qlen, item_slots, tails, taps, width);
}

}  // extern "C"
