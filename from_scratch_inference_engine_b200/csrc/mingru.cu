// minGRU: an element-wise recurrence; gate and candidate of a token come from that token's
// projections alone, never from the state.
//
//   proj[t] = [ a | u | g ]  (three blocks of `width` columns: the product's result, biases added)
//   z = sigmoid(a);   cand = (u < 0) ? sigmoid(u) : u + 0.5
//   S_t = (1 - z) S_{t-1} + z cand            (S: float32 [width] in the request's state slot)
//   out[t] = T( S_t * silu(g) )
//
// Gates, candidate, state and the gated output are 32-bit whatever the storage type T of proj and
// out.  A request's tokens are walked in order by one thread per channel.  Long prompts run
// chunk-parallel: the recurrence S -> A S + B composes, so every chunk of a request first folds
// its own tokens into (A, B) = (prod (1 - z), the state it would reach from zero), a chain kernel
// turns those into the state at each chunk's start, and every chunk runs again from there.
#include "common.cuh"
#include <math.h>

namespace fsie {

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

__device__ __forceinline__ void mingru_gates(float a, float u, float& z, float& cand) {
    z = sigmoid_f(a);
    cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
}

// mode 0: walk a whole request from its stored state, write outputs and the new state
// mode 1: a segment from zero: leave (A, B) in seg_ab[seg][2][width], no outputs
// mode 2: a segment from seg_start[seg][width]: write outputs; the request's last segment writes the state
template <typename T, int MODE>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, int ld, int width,
                                   const int* __restrict__ item_qstart, const int* __restrict__ item_qlen,
                                   const int* __restrict__ item_slots, const int* __restrict__ seg_item,
                                   const int* __restrict__ seg_row0, int seg_tokens,
                                   float* __restrict__ state, float* __restrict__ seg_ab,
                                   const float* __restrict__ seg_start, T* __restrict__ out) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int unit = blockIdx.y;
    const int item = MODE == 0 ? unit : seg_item[unit];
    grid_dependency_wait();
    grid_dependents_go();
    const int slot = item_slots[item];
    if (slot < 0 || c >= width) return;            // a padding entry of a fixed-size batch
    const int qlen = item_qlen[item];
    const int first = MODE == 0 ? 0 : seg_row0[unit];
    const int count = MODE == 0 ? qlen : min(seg_tokens, qlen - first);
    if (count <= 0) return;
    const T* row = proj + (size_t)(item_qstart[item] + first) * ld + c;
    float s = 0.f, carry = 1.f;
    if (MODE == 0) s = state[(size_t)slot * width + c];
    if (MODE == 2) s = seg_start[(size_t)unit * width + c];
    T* o = MODE == 1 ? nullptr : out + (size_t)(item_qstart[item] + first) * width + c;
    // eight tokens' values are asked for before the first is used: the loads do not depend on the
    // recurrence, only the sums do
    constexpr int AHEAD = 8;
    for (int t0 = 0; t0 < count; t0 += AHEAD) {
        T av[AHEAD], uv[AHEAD], gv[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const bool in = t0 + j < count;
            const T* r = row + (size_t)(in ? j : 0) * ld;
            av[j] = r[0];
            uv[j] = r[width];
            if (MODE != 1) gv[j] = r[2 * width];
        }
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            if (t0 + j >= count) break;
            float z, cand;
            mingru_gates(to_float(av[j]), to_float(uv[j]), z, cand);
            s = (1.0f - z) * s + z * cand;
            if (MODE == 1) {
                carry *= 1.0f - z;
            } else {
                const float g = to_float(gv[j]);
                o[0] = from_float<T>(s * (g / (1.0f + expf(-g))));
                o += width;
            }
        }
        row += (size_t)AHEAD * ld;
    }
    if (MODE == 0 || (MODE == 2 && first + count >= qlen)) state[(size_t)slot * width + c] = s;
    if (MODE == 1) {
        seg_ab[((size_t)unit * 2) * width + c] = carry;
        seg_ab[((size_t)unit * 2 + 1) * width + c] = s;
    }
}

// The state at the start of every segment: segments of a request follow one another in the list,
// the first starts from the stored state.
__global__ void mingru_chain_kernel(const int* __restrict__ item_slots, const int* __restrict__ seg_item,
                                    const int* __restrict__ seg_row0, int num_segs, int width,
                                    const float* __restrict__ state, const float* __restrict__ seg_ab,
                                    float* __restrict__ seg_start) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    grid_dependency_wait();
    grid_dependents_go();
    float s = 0.f;
    // eight segments' (A, B), slots and first rows are asked for before the chain through them runs
    constexpr int AHEAD = 8;
    for (int seg0 = 0; seg0 < num_segs; seg0 += AHEAD) {
        float a[AHEAD], b[AHEAD];
        int slot[AHEAD], row0[AHEAD];
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            const int seg = min(seg0 + j, num_segs - 1);
            a[j] = seg_ab[((size_t)seg * 2) * width + c];
            b[j] = seg_ab[((size_t)seg * 2 + 1) * width + c];
            slot[j] = item_slots[seg_item[seg]];
            row0[j] = seg_row0[seg];
        }
#pragma unroll
        for (int j = 0; j < AHEAD; ++j) {
            if (seg0 + j >= num_segs) break;
            if (slot[j] < 0) continue;
            if (row0[j] == 0) s = state[(size_t)slot[j] * width + c];
            seg_start[(size_t)(seg0 + j) * width + c] = s;
            s = a[j] * s + b[j];
        }
    }
}

template <typename T>
static int mingru_launch(const void* proj, int ld, int width, const int* item_qstart, const int* item_qlen,
                         const int* item_slots, int items, const int* seg_item, const int* seg_row0,
                         int num_segs, int seg_tokens, float* state, float* seg_ab, float* seg_start,
                         void* out, cudaStream_t stream) {
    const int threads = width >= 128 ? 128 : 64;
    const unsigned cols = (unsigned)((width + threads - 1) / threads);
    if (num_segs <= 0)
        return launch_dependent(mingru_scan_kernel<T, 0>, dim3(cols, items), dim3(threads), 0, stream,
                                (const T*)proj, ld, width, item_qstart, item_qlen, item_slots, seg_item,
                                seg_row0, seg_tokens, state, seg_ab, (const float*)seg_start, (T*)out);
    int rc = launch_dependent(mingru_scan_kernel<T, 1>, dim3(cols, num_segs), dim3(threads), 0, stream,
                              (const T*)proj, ld, width, item_qstart, item_qlen, item_slots, seg_item,
                              seg_row0, seg_tokens, state, seg_ab, (const float*)seg_start, (T*)out);
    if (rc) return rc;
    rc = launch_dependent(mingru_chain_kernel, dim3(cols), dim3(threads), 0, stream, item_slots, seg_item,
                          seg_row0, num_segs, width, (const float*)state, (const float*)seg_ab, seg_start);
    if (rc) return rc;
    return launch_dependent(mingru_scan_kernel<T, 2>, dim3(cols, num_segs), dim3(threads), 0, stream,
                            (const T*)proj, ld, width, item_qstart, item_qlen, item_slots, seg_item,
                            seg_row0, seg_tokens, state, seg_ab, (const float*)seg_start, (T*)out);
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// proj [tokens, ld] with the three blocks at columns 0, width, 2 width; out [tokens, width];
// state float32 [slots, width].  num_segs = 0: one walk per request.  Else the requests are cut
// into segments of seg_tokens tokens (seg_item / seg_row0, in order, a request's segments together),
// seg_ab holds 2 * num_segs * width floats and seg_start num_segs * width.
int fsie_mingru_scan(const void* proj, int ld, int width, const int* item_qstart, const int* item_qlen,
                     const int* item_slots, int items, const int* seg_item, const int* seg_row0,
                     int num_segs, int seg_tokens, float* state, float* seg_ab, float* seg_start,
                     void* out, int dtype, cudaStream_t stream) {
    if (items <= 0) return 0;
    if (width <= 0 || ld < 3 * width || items > 65535 || num_segs > 65535) return ERR_BAD_ARGUMENT;
    if (num_segs > 0 && (!seg_item || !seg_row0 || !seg_ab || !seg_start || seg_tokens <= 0))
        return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return mingru_launch<float>(proj, ld, width, item_qstart, item_qlen, item_slots, items, seg_item,
                                    seg_row0, num_segs, seg_tokens, state, seg_ab, seg_start, out, stream);
    return mingru_launch<bf16>(proj, ld, width, item_qstart, item_qlen, item_slots, items, seg_item,
                               seg_row0, num_segs, seg_tokens, state, seg_ab, seg_start, out, stream);
}

}  // extern "C"
