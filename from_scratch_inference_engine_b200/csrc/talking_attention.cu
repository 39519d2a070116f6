// Attention whose softmax weights are mixed across heads ("talking heads"), over a sliding
// window that also keeps the first tokens of the sequence, fed by projections that pass a
// short causal convolution, whole-projection RMS norms and an interleaved rotation.
//
//   prepare   u = conv(projected q | k | v)              y_t = sum_j w[:, j] u_{t - taps + 1 + j}
//             q = rot(rms(u_q) * w_q)   k = rot(rms(u_k) * w_k)     rms over the WHOLE projection
//             v_head = u_v,head / sqrt(mean(u_v,head^2) + eps)
//             q -> a 32-bit buffer; k, v -> the pages of the cache
//   tails     the last taps - 1 projected rows of every request -> its state slot
//   attend    s_h(i, j) = (q_h,i . k_g(h),j) * scale  for visible j:
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

// ------------------------------------------------------------------------------ attend
constexpr int TA_KEYS = 64;        // keys of one tile
constexpr int TA_WARPS = 8;
constexpr int TA_MAX_ROWS = 64;    // (token, head) rows of one block: 8 per warp

struct TalkingArgs {
    const float* q; const void* k_pages; const void* v_pages; long long page_stride; int page_size;
    const int* block_tables; int table_stride; const int* tile_item; const int* tile_row0;
    const int* item_qstart; const int* item_qlen; const int* item_pos0; const int* item_slots;
    const float* talk;
    void* out; int heads, kv_heads, dim, vdim, window, keep_first, tile_tokens; float scale; int* error;
};

// One block per tile of `tile_tokens` consecutive tokens of one request, all heads: row r =
// token * heads + head.  Warp w owns rows w, w + 8, ...  The visible keys of the tile are the kept
// first tokens below the window, then the window of its first token up to its last token; they
// are walked twice in tiles of TA_KEYS: once for every row's maximum and sum, once to form the
// normalised weights of all heads, mix them and apply them to the values.
template <typename T, int VC>
__global__ void __launch_bounds__(TA_WARPS * 32)
talking_attention_kernel(const TalkingArgs a) {
    extern __shared__ float smem[];
    const int H = a.heads, G = a.kv_heads, dim = a.dim, vdim = a.vdim;
    const int group = H / G;
    const int tile = blockIdx.x;
    const int item = a.tile_item[tile], tok0 = a.tile_row0[tile];
    if (a.item_slots[item] < 0) return;                 // a padding entry of a fixed-size batch
    const int qlen = a.item_qlen[item];
    const int n_tok = min(a.tile_tokens, qlen - tok0);
    if (n_tok <= 0) return;
    const int R = n_tok * H;
    const int p_first = a.item_pos0[item] + tok0, p_last = p_first + n_tok - 1;
    const int lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int kept = min(a.keep_first, lo);             // kept first tokens that lie below the window
    const int n_keys = kept + (p_last - lo + 1);
    const int kv_ld = max(dim, vdim) + 1;

    float* qs = smem;                                   // [rows][dim]
    float* kv = qs + TA_MAX_ROWS * dim;                 // [TA_KEYS][kv_ld]
    float* P = kv + TA_KEYS * kv_ld;                    // [rows][TA_KEYS]
    float* P2 = P + TA_MAX_ROWS * TA_KEYS;              // [rows][TA_KEYS]
    float* talk = P2 + TA_MAX_ROWS * TA_KEYS;           // [H][H]
    int* key_page = reinterpret_cast<int*>(talk + H * H);   // [TA_KEYS]
    int* key_off = key_page + TA_KEYS;                  // [TA_KEYS]

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* k_pages = reinterpret_cast<const T*>(a.k_pages);
    const T* v_pages = reinterpret_cast<const T*>(a.v_pages);
    const int* table = a.block_tables + (size_t)item * a.table_stride;

    const size_t q_row0 = (size_t)(a.item_qstart[item] + tok0) * H * dim;
    for (int idx = threadIdx.x; idx < R * dim; idx += blockDim.x) qs[idx] = a.q[q_row0 + idx];
    for (int idx = threadIdx.x; idx < H * H; idx += blockDim.x) talk[idx] = a.talk[idx];

    float row_max[TA_MAX_ROWS / TA_WARPS], row_sum[TA_MAX_ROWS / TA_WARPS];
    float acc[TA_MAX_ROWS / TA_WARPS][VC];
#pragma unroll
    for (int k = 0; k < TA_MAX_ROWS / TA_WARPS; ++k) {
        row_max[k] = -INFINITY;
        row_sum[k] = 0.f;
#pragma unroll
        for (int c = 0; c < VC; ++c) acc[k][c] = 0.f;
    }

    for (int pass = 0; pass < 2; ++pass) {
        for (int u0 = 0; u0 < n_keys; u0 += TA_KEYS) {
            const int n = min(TA_KEYS, n_keys - u0);
            __syncthreads();                             // the tile before is done with kv, P, P2
            if (threadIdx.x < TA_KEYS) {
                int page = -1, off = 0;
                if ((int)threadIdx.x < n) {
                    const int u = u0 + threadIdx.x;
                    const int j = u < kept ? u : lo + (u - kept);
                    page = table[j / a.page_size];
                    off = j - (j / a.page_size) * a.page_size;
                    if (page < 0) atomicExch(a.error, 3);      // a visible key's page was given back
                }
                key_page[threadIdx.x] = page;
                key_off[threadIdx.x] = off;
            }
            for (int g = 0; g < G; ++g) {
                __syncthreads();                         // key_page is written; kv is free again
                for (int idx = threadIdx.x; idx < n * dim; idx += blockDim.x) {
                    const int jj = idx / dim, d = idx - jj * dim;
                    const int page = key_page[jj];
                    kv[jj * kv_ld + d] = page < 0 ? 0.f : to_float(
                        k_pages[page * a.page_stride + ((size_t)g * a.page_size + key_off[jj]) * dim + d]);
                }
                __syncthreads();
#pragma unroll
                for (int k = 0; k < TA_MAX_ROWS / TA_WARPS; ++k) {
                    const int r = warp + TA_WARPS * k;
                    if (r >= R) continue;
                    const int i = r / H, h = r - i * H;
                    if (h / group != g) continue;
                    const int p_i = p_first + i;
                    const float* qr = qs + r * dim;
                    float s0 = 0.f, s1 = 0.f;
                    const float* k0 = kv + lane * kv_ld;
                    const float* k1 = kv + (lane + 32) * kv_ld;
                    for (int d = 0; d < dim; ++d) {
                        const float qd = qr[d];
                        s0 += qd * k0[d];
                        s1 += qd * k1[d];
                    }
                    const int ua = u0 + lane, ub = u0 + lane + 32;
                    const int ja = ua < kept ? ua : lo + (ua - kept);
                    const int jb = ub < kept ? ub : lo + (ub - kept);
                    const bool see_a = lane < n && ja <= p_i &&
                        (a.window <= 0 || p_i - ja < a.window || ja < a.keep_first);
                    const bool see_b = lane + 32 < n && jb <= p_i &&
                        (a.window <= 0 || p_i - jb < a.window || jb < a.keep_first);
                    s0 = see_a ? s0 * a.scale : -INFINITY;
                    s1 = see_b ? s1 * a.scale : -INFINITY;
                    if (pass == 0) {
                        const float m_new = fmaxf(row_max[k], warp_max(fmaxf(s0, s1)));
                        if (m_new > -INFINITY) {
                            const float e = (see_a ? expf(s0 - m_new) : 0.f) + (see_b ? expf(s1 - m_new) : 0.f);
                            row_sum[k] = row_sum[k] * expf(row_max[k] - m_new) + warp_sum(e);
                            row_max[k] = m_new;
                        }
                    } else {
                        const float inv = 1.0f / row_sum[k];
                        P[r * TA_KEYS + lane] = see_a ? expf(s0 - row_max[k]) * inv : 0.f;
                        P[r * TA_KEYS + lane + 32] = see_b ? expf(s1 - row_max[k]) * inv : 0.f;
                    }
                }
            }
            if (pass == 0) continue;
            __syncthreads();                             // P holds every head's weights of this tile
            for (int idx = threadIdx.x; idx < R * TA_KEYS; idx += blockDim.x) {
                const int r = idx / TA_KEYS, jj = idx - r * TA_KEYS;
                const int i = r / H, h = r - i * H;
                const float* mix = talk + h * H;
                const float* col = P + (size_t)i * H * TA_KEYS + jj;
                float m = 0.f;
                for (int g2 = 0; g2 < H; ++g2) m += mix[g2] * col[g2 * TA_KEYS];
                P2[idx] = m;
            }
            for (int g = 0; g < G; ++g) {
                __syncthreads();                         // P2 is written; kv is free again
                for (int idx = threadIdx.x; idx < n * vdim; idx += blockDim.x) {
                    const int jj = idx / vdim, d = idx - jj * vdim;
                    const int page = key_page[jj];
                    kv[jj * kv_ld + d] = page < 0 ? 0.f : to_float(
                        v_pages[page * a.page_stride + ((size_t)g * a.page_size + key_off[jj]) * vdim + d]);
                }
                __syncthreads();
#pragma unroll
                for (int k = 0; k < TA_MAX_ROWS / TA_WARPS; ++k) {
                    const int r = warp + TA_WARPS * k;
                    if (r >= R) continue;
                    const int h = r % H;
                    if (h / group != g) continue;
                    const float* w = P2 + r * TA_KEYS;
                    for (int jj = 0; jj < n; ++jj) {
                        const float p = w[jj];
                        const float* vr = kv + jj * kv_ld;
#pragma unroll
                        for (int c = 0; c < VC; ++c) {
                            const int col = lane + 32 * c;
                            if (col < vdim) acc[k][c] += p * vr[col];
                        }
                    }
                }
            }
        }
    }
    T* out = reinterpret_cast<T*>(a.out) + (size_t)(a.item_qstart[item] + tok0) * H * vdim;
#pragma unroll
    for (int k = 0; k < TA_MAX_ROWS / TA_WARPS; ++k) {
        const int r = warp + TA_WARPS * k;
        if (r >= R) continue;
#pragma unroll
        for (int c = 0; c < VC; ++c) {
            const int col = lane + 32 * c;
            if (col < vdim) out[(size_t)r * vdim + col] = from_float<T>(acc[k][c]);
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
#define FSIE_PREPARE(T)                                                                          \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            cudaFuncSetAttribute(conv_norm_rotate_kernel<T>,                                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        conv_norm_rotate_kernel<T><<<tokens, threads, smem, stream>>>(                           \
            (const T*)proj, ld, items, item_qstart, item_pos0, item_slots, tails, conv_w, taps,  \
            q_gain, k_gain, cos_sin, table_len, rot_dims, slot_of, (T*)k_pages, (T*)v_pages,     \
            page_stride, page_size, q_out, heads, kv_heads, dim, vdim, has_kv, eps, error);      \
    } while (0)
    if (dtype == DTYPE_F32) FSIE_PREPARE(float);
    else FSIE_PREPARE(bf16);
#undef FSIE_PREPARE
    return FSIE_LAUNCH_CHECK();
}

int fsie_conv_tails(const void* proj, int ld, const int* item_qstart, const int* item_qlen,
                    const int* item_slots, int items, float* tails, int taps, int width, int dtype,
                    cudaStream_t stream) {
    if (items <= 0 || taps <= 1) return 0;
    if (dtype == DTYPE_F32)
        conv_tails_kernel<float><<<items, 256, 0, stream>>>((const float*)proj, ld, item_qstart,
                                                           item_qlen, item_slots, tails, taps, width);
    else
        conv_tails_kernel<bf16><<<items, 256, 0, stream>>>((const bf16*)proj, ld, item_qstart,
                                                          item_qlen, item_slots, tails, taps, width);
    return FSIE_LAUNCH_CHECK();
}

// Tokens of one tile for a model with `heads` heads (rows of a block: tokens * heads <= 64).
int fsie_talking_attention_tile_tokens(int heads) {
    if (heads <= 0 || heads > TA_MAX_ROWS) return 0;
    const int tokens = TA_MAX_ROWS / heads;
    return tokens > 16 ? 16 : tokens;
}

int fsie_talking_attention(const float* q, const void* k_pages, const void* v_pages,
                           long long page_stride, int page_size, const int* block_tables,
                           int table_stride, const int* tile_item, const int* tile_row0, int num_tiles,
                           const int* item_qstart, const int* item_qlen, const int* item_pos0,
                           const int* item_slots, const float* talk, void* out, int heads, int kv_heads, int dim, int vdim,
                           int window, int keep_first, int tile_tokens, float scale, int dtype,
                           int* error, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || tile_tokens <= 0 ||
        tile_tokens * heads > TA_MAX_ROWS || window < 0 || keep_first < 0)
        return ERR_BAD_ARGUMENT;
    if (vdim > 256) return ERR_UNSUPPORTED;
    const int kv_ld = (dim > vdim ? dim : vdim) + 1;
    const size_t smem = ((size_t)TA_MAX_ROWS * dim + (size_t)TA_KEYS * kv_ld +
                         2 * (size_t)TA_MAX_ROWS * TA_KEYS + (size_t)heads * heads) * sizeof(float) +
                        2 * TA_KEYS * sizeof(int);
    if (smem > 220 * 1024) return ERR_UNSUPPORTED;
    TalkingArgs a = {q, k_pages, v_pages, page_stride, page_size, block_tables, table_stride,
                     tile_item, tile_row0, item_qstart, item_qlen, item_pos0, item_slots, talk, out,
                     heads,
                     kv_heads, dim, vdim, window, keep_first, tile_tokens, scale, error};
    const int vc = (vdim + 31) / 32;
#define FSIE_ATTEND(T, VC)                                                                       \
    do {                                                                                         \
        cudaFuncSetAttribute(talking_attention_kernel<T, VC>,                                    \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
        talking_attention_kernel<T, VC><<<num_tiles, TA_WARPS * 32, smem, stream>>>(a);          \
    } while (0)
#define FSIE_ATTEND_BY_SIZE(T)                                                                   \
    do {                                                                                         \
        if (vc <= 1) FSIE_ATTEND(T, 1);                                                          \
        else if (vc <= 2) FSIE_ATTEND(T, 2);                                                     \
        else if (vc <= 4) FSIE_ATTEND(T, 4);                                                     \
        else FSIE_ATTEND(T, 8);                                                                  \
    } while (0)
    if (dtype == DTYPE_F32) FSIE_ATTEND_BY_SIZE(float);
    else FSIE_ATTEND_BY_SIZE(bf16);
#undef FSIE_ATTEND_BY_SIZE
#undef FSIE_ATTEND
    return FSIE_LAUNCH_CHECK();
}

}  // extern "C"
