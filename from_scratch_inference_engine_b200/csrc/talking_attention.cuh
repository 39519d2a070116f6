// Softmax attention whose normalised weights are mixed across heads before they meet the
// values, over a sliding window that also keeps the first tokens of the sequence.
//
//   s_h(i, j) = (q_h,i . k_g(h),j) * scale   for visible j:
//                   j <= i and (window == 0 or i - j < window or j < keep_first)
//   p_h = softmax_j s_h            p'_h = sum_h' talk[h, h'] p_h'
//   o_h,i = sum_j p'_h(i, j) v_g(h),j                      g(h) = h / (heads / kv_heads)
//
// The mixing needs every head's FINISHED softmax at the same (i, j), so one block takes a tile of
// consecutive tokens of one request with all heads and walks the visible keys twice: once for
// every row's maximum and sum, once to form the weights, mix them and apply them to the values.
// Scores, softmax, mixed weights and outputs are 32-bit arithmetic on the CUDA cores whatever the
// storage type T of the pages.  A tile whose keys are many and whose tokens are few (decoding)
// is split over several blocks by key range: a first launch leaves every range's maximum and
// sum, a second combines them, applies its own range and leaves a partial output, a third adds
// the partial outputs in a fixed order.
//
// Included by one source file per storage type, which instantiates `talking_attention_launch`.
#pragma once

#include "common.cuh"

namespace fsie {

constexpr int TA_WARPS = 8;
constexpr int TA_ROWS = 64;        // (token, head) rows a block holds at most: 8 per warp

struct TalkingArgs {
    const float* q; const void* k_pages; const void* v_pages; long long page_stride; int page_size;
    const int* block_tables; int table_stride; const int* tile_item; const int* tile_row0;
    const int* item_qstart; const int* item_qlen; const int* item_pos0; const int* item_slots;
    const float* talk; void* out;
    int heads, kv_heads, dim, vdim, window, keep_first, tile_tokens;
    float scale; int* error;
    int nsplit, mode;              // mode 0: both walks, out; 1: first walk, part_stats; 2: second walk, part_out
    float* part_stats;             // [tiles][nsplit][TA_ROWS][2]
    float* part_out;               // [nsplit][tokens][heads * vdim]
    int tokens;
};

__device__ __forceinline__ void load2(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
}
__device__ __forceinline__ void load2(const bf16* p, float& a, float& b) {
    const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    a = v.x; b = v.y;
}

// sizes of the shared-memory layout, the same on host and device
struct TalkingLayout {
    int dim8, vdim8, q_ld, kv_ld;
    size_t q_bytes, kv_bytes, p_bytes, talk_bytes, total;
    __host__ __device__ TalkingLayout(int heads, int kv_heads, int dim, int vdim, int key_tile,
                                      int elem_bytes) {
        dim8 = (dim + 7) & ~7;
        vdim8 = (vdim + 7) & ~7;
        q_ld = dim8 + 4;
        kv_ld = (dim8 > vdim8 ? dim8 : vdim8) + 16 / elem_bytes;     // rows 16 bytes apart in banks
        q_bytes = (size_t)TA_ROWS * q_ld * sizeof(float);
        kv_bytes = (size_t)kv_heads * key_tile * kv_ld * elem_bytes;
        p_bytes = (size_t)TA_ROWS * key_tile * sizeof(float);
        talk_bytes = (((size_t)heads * heads * sizeof(float)) + 15) & ~(size_t)15;
        total = q_bytes + kv_bytes + 2 * p_bytes + talk_bytes + 2 * key_tile * sizeof(int);
    }
};

// One tile of keys (or values) of every key/value head from the pages into shared memory
// [g][key][ld], zero beyond `width` and for keys without a page: a warp copies a row, 16 bytes
// per lane where the rows allow it.
template <typename T>
__device__ __forceinline__ void copy_tile(T* __restrict__ dst, const T* __restrict__ pages,
                                          const int* key_page, const int* key_off, int G, int keys,
                                          int width, int width8, int ld, long long page_stride,
                                          int page_size, int warp, int lane) {
    constexpr int PER = 16 / (int)sizeof(T);                 // elements of one 16-byte piece
    const bool wide = width % PER == 0 && page_stride % PER == 0 &&
                      (reinterpret_cast<uintptr_t>(pages) & 15) == 0;
    for (int row = warp; row < G * keys; row += TA_WARPS) {
        const int g = row / keys, jj = row - g * keys;
        const int page = key_page[jj];
        T* to = dst + (size_t)row * ld;
        const T* from = page < 0 ? nullptr :
            pages + page * page_stride + ((size_t)g * page_size + key_off[jj]) * width;
        if (wide) {
            for (int piece = lane; piece * PER < width8; piece += 32) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (from && piece * PER < width) v = *reinterpret_cast<const uint4*>(from + piece * PER);
                *reinterpret_cast<uint4*>(to + piece * PER) = v;
            }
        } else {
            for (int d = lane; d < width8; d += 32)
                to[d] = (from && d < width) ? from[d] : from_float<T>(0.f);
        }
    }
}

// Warp w owns heads w, w + 8, ... (HS = 8 / TOK of them at most) and, of each, the tile's TOK
// tokens: rows that share their keys and values, so one load of a key or value serves TOK rows.
// Lane l owns keys l (+ 32) of a tile for the scores and value columns 2 l, 2 l + 1 (+ 64 c).
template <typename T, int TOK, int VC2, int KPL>
__global__ void __launch_bounds__(TA_WARPS * 32) talking_attention_kernel(const TalkingArgs a) {
    constexpr int HS = 8 / TOK;
    constexpr int TK = 32 * KPL;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.heads, G = a.kv_heads, dim = a.dim, vdim = a.vdim;
    const int group = H / G;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int item = a.tile_item[tile], tok0 = a.tile_row0[tile];
    if (a.item_slots[item] < 0) return;                 // a padding entry of a fixed-size batch
    const int n_tok = min(TOK, a.item_qlen[item] - tok0);
    if (n_tok <= 0) return;
    const int R = n_tok * H;
    const int p_first = a.item_pos0[item] + tok0, p_last = p_first + n_tok - 1;
    const int lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int kept = min(a.keep_first, lo);             // kept first tokens that lie below the window
    const int n_keys = kept + (p_last - lo + 1);
    const int key_tiles = (n_keys + TK - 1) / TK;
    const int per_split = (key_tiles + a.nsplit - 1) / a.nsplit;
    const int u_begin = min(n_keys, split * per_split * TK);
    const int u_end = min(n_keys, (split + 1) * per_split * TK);

    const TalkingLayout L(H, G, dim, vdim, TK, (int)sizeof(T));
    float* qs = reinterpret_cast<float*>(smem_raw);
    T* kv = reinterpret_cast<T*>(smem_raw + L.q_bytes);
    float* P = reinterpret_cast<float*>(smem_raw + L.q_bytes + L.kv_bytes);
    float* P2 = P + TA_ROWS * TK;
    float* talk = P2 + TA_ROWS * TK;
    int* key_page = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(talk) + L.talk_bytes);
    int* key_off = key_page + TK;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* k_pages = reinterpret_cast<const T*>(a.k_pages);
    const T* v_pages = reinterpret_cast<const T*>(a.v_pages);
    const int* table = a.block_tables + (size_t)item * a.table_stride;
    const int token0 = a.item_qstart[item] + tok0;

    // q rows [tok * H + h], zero beyond dim and beyond the tile's tokens
    for (int idx = threadIdx.x; idx < TOK * H * L.dim8; idx += blockDim.x) {
        const int r = idx / L.dim8, d = idx - r * L.dim8;
        qs[r * L.q_ld + d] = (r < R && d < dim) ? a.q[((size_t)token0 * H + r) * dim + d] : 0.f;
    }
    for (int idx = threadIdx.x; idx < H * H; idx += blockDim.x) talk[idx] = a.talk[idx];

    float row_max[HS][TOK], row_sum[HS][TOK], acc[HS][TOK][VC2][2];
#pragma unroll
    for (int hs = 0; hs < HS; ++hs)
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            row_max[hs][t] = -INFINITY;
            row_sum[hs][t] = 0.f;
#pragma unroll
            for (int c = 0; c < VC2; ++c) acc[hs][t][c][0] = acc[hs][t][c][1] = 0.f;
        }

    if (a.mode == 2) {
        // maximum and sum over all key ranges, from what the first launch left
        __syncthreads();
        const float* stats = a.part_stats + (size_t)tile * a.nsplit * TA_ROWS * 2;
#pragma unroll
        for (int hs = 0; hs < HS; ++hs) {
            const int h = warp + TA_WARPS * hs;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                if (h >= H || t >= n_tok) continue;
                const int r = t * H + h;
                float m = -INFINITY;
                for (int s = 0; s < a.nsplit; ++s) m = fmaxf(m, stats[((size_t)s * TA_ROWS + r) * 2]);
                float l = 0.f;
                for (int s = 0; s < a.nsplit; ++s) {
                    const float ms = stats[((size_t)s * TA_ROWS + r) * 2];
                    if (ms > -INFINITY) l += stats[((size_t)s * TA_ROWS + r) * 2 + 1] * expf(ms - m);
                }
                row_max[hs][t] = m;
                row_sum[hs][t] = l;
            }
        }
    }

    const int first_pass = a.mode == 2 ? 1 : 0, last_pass = a.mode == 1 ? 0 : 1;
    for (int pass = first_pass; pass <= last_pass; ++pass) {
        for (int u0 = u_begin; u0 < u_end; u0 += TK) {
            const int n = min(TK, u_end - u0);
            __syncthreads();                             // the tile before is done with kv, P, P2
            if (threadIdx.x < TK) {
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
            __syncthreads();
            // keys of every key/value head: [g][key][dim8], zero beyond dim and beyond the tile
            copy_tile<T>(kv, k_pages, key_page, key_off, G, TK, dim, L.dim8, L.kv_ld, a.page_stride,
                         a.page_size, warp, lane);
            __syncthreads();
#pragma unroll
            for (int hs = 0; hs < HS; ++hs) {
                const int h = warp + TA_WARPS * hs;
                if (h >= H) continue;
                const int g = h / group;
                float s[TOK][KPL];
#pragma unroll
                for (int t = 0; t < TOK; ++t)
#pragma unroll
                    for (int kp = 0; kp < KPL; ++kp) s[t][kp] = 0.f;
                for (int d = 0; d < L.dim8; d += 8) {
                    float kk[KPL][8];
#pragma unroll
                    for (int kp = 0; kp < KPL; ++kp)
                        load8(kv + ((size_t)g * TK + lane + 32 * kp) * L.kv_ld + d, kk[kp]);
#pragma unroll
                    for (int t = 0; t < TOK; ++t) {
                        float qq[8];
                        load8(qs + (t * H + h) * L.q_ld + d, qq);
#pragma unroll
                        for (int kp = 0; kp < KPL; ++kp)
#pragma unroll
                            for (int e = 0; e < 8; ++e) s[t][kp] += qq[e] * kk[kp][e];
                    }
                }
#pragma unroll
                for (int t = 0; t < TOK; ++t) {
                    if (t >= n_tok) continue;
                    const int p_i = p_first + t;
                    bool see[KPL];
                    float tile_max = -INFINITY;
#pragma unroll
                    for (int kp = 0; kp < KPL; ++kp) {
                        const int u = u0 + lane + 32 * kp;
                        const int j = u < kept ? u : lo + (u - kept);
                        see[kp] = lane + 32 * kp < n && j <= p_i &&
                            (a.window <= 0 || p_i - j < a.window || j < a.keep_first);
                        s[t][kp] = see[kp] ? s[t][kp] * a.scale : -INFINITY;
                        tile_max = fmaxf(tile_max, s[t][kp]);
                    }
                    if (pass == 0) {
                        const float m_new = fmaxf(row_max[hs][t], warp_max(tile_max));
                        if (m_new > -INFINITY) {
                            float e = 0.f;
#pragma unroll
                            for (int kp = 0; kp < KPL; ++kp) e += see[kp] ? expf(s[t][kp] - m_new) : 0.f;
                            row_sum[hs][t] = row_sum[hs][t] * expf(row_max[hs][t] - m_new) + warp_sum(e);
                            row_max[hs][t] = m_new;
                        }
                    } else {
                        const float inv = 1.0f / row_sum[hs][t];
#pragma unroll
                        for (int kp = 0; kp < KPL; ++kp)
                            P[(t * H + h) * TK + lane + 32 * kp] =
                                see[kp] ? expf(s[t][kp] - row_max[hs][t]) * inv : 0.f;
                    }
                }
            }
            if (pass == 0) continue;
            __syncthreads();                             // P holds every head's weights of this tile
            for (int idx = threadIdx.x; idx < R * TK; idx += blockDim.x) {
                const int r = idx / TK, jj = idx - r * TK;
                const int t = r / H, h = r - t * H;
                const float* mix = talk + h * H;
                const float* col = P + (size_t)t * H * TK + jj;
                float m = 0.f;
                for (int h2 = 0; h2 < H; ++h2) m += mix[h2] * col[h2 * TK];
                P2[idx] = m;
            }
            // values of every key/value head: [g][key][vdim8], zero beyond vdim and beyond the tile
            copy_tile<T>(kv, v_pages, key_page, key_off, G, TK, vdim, L.vdim8, L.kv_ld, a.page_stride,
                         a.page_size, warp, lane);
            __syncthreads();
#pragma unroll
            for (int hs = 0; hs < HS; ++hs) {
                const int h = warp + TA_WARPS * hs;
                if (h >= H) continue;
                const T* vg = kv + (size_t)(h / group) * TK * L.kv_ld;
                for (int jj = 0; jj < TK; jj += 4) {
                    if (jj >= n) break;
                    float4 p[TOK];
#pragma unroll
                    for (int t = 0; t < TOK; ++t)
                        p[t] = t < n_tok ? *reinterpret_cast<const float4*>(P2 + (t * H + h) * TK + jj)
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int c = 0; c < VC2; ++c) {
                        const int col = 2 * lane + 64 * c;
                        if (col >= L.vdim8) continue;
                        float v[4][2];
#pragma unroll
                        for (int x = 0; x < 4; ++x) load2(vg + (size_t)(jj + x) * L.kv_ld + col, v[x][0], v[x][1]);
#pragma unroll
                        for (int t = 0; t < TOK; ++t) {
                            acc[hs][t][c][0] += p[t].x * v[0][0] + p[t].y * v[1][0] + p[t].z * v[2][0] + p[t].w * v[3][0];
                            acc[hs][t][c][1] += p[t].x * v[0][1] + p[t].y * v[1][1] + p[t].z * v[2][1] + p[t].w * v[3][1];
                        }
                    }
                }
            }
        }
    }

    if (a.mode == 1) {
        float* stats = a.part_stats + ((size_t)tile * a.nsplit + split) * TA_ROWS * 2;
#pragma unroll
        for (int hs = 0; hs < HS; ++hs) {
            const int h = warp + TA_WARPS * hs;
#pragma unroll
            for (int t = 0; t < TOK; ++t) {
                if (h >= H || t >= n_tok || lane != 0) continue;
                stats[(t * H + h) * 2] = row_max[hs][t];
                stats[(t * H + h) * 2 + 1] = row_sum[hs][t];
            }
        }
        return;
    }
#pragma unroll
    for (int hs = 0; hs < HS; ++hs) {
        const int h = warp + TA_WARPS * hs;
        if (h >= H) continue;
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
            if (t >= n_tok) continue;
            const size_t at = ((size_t)(token0 + t) * H + h) * vdim;
#pragma unroll
            for (int c = 0; c < VC2; ++c)
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int col = 2 * lane + 64 * c + x;
                    if (col >= vdim) continue;
                    if (a.mode == 0) reinterpret_cast<T*>(a.out)[at + col] = from_float<T>(acc[hs][t][c][x]);
                    else a.part_out[(size_t)split * a.tokens * H * vdim + at + col] = acc[hs][t][c][x];
                }
        }
    }
}

// out = the partial outputs of the key ranges added in order
template <typename T>
__global__ void talking_attention_merge_kernel(const float* __restrict__ part, T* __restrict__ out,
                                               long long count, int nsplit) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        float v = 0.f;
        for (int s = 0; s < nsplit; ++s) v += part[(size_t)s * count + i];
        out[i] = from_float<T>(v);
    }
}

// keys of one tile (64 or 32) that fit the shared memory for these sizes; 0: none does
inline int talking_key_tile(int heads, int kv_heads, int dim, int vdim, int elem_bytes) {
    const size_t limits[2] = {110 * 1024, 220 * 1024};   // two blocks on an SM, else one
    for (size_t limit : limits)
        for (int tile = 64; tile >= 32; tile /= 2)
            if (TalkingLayout(heads, kv_heads, dim, vdim, tile, elem_bytes).total <= limit) return tile;
    return 0;
}

template <typename T, int TOK, int VC2>
int talking_attention_launch_tile(const TalkingArgs& a, int num_tiles, int key_tile, size_t smem,
                                  cudaStream_t stream) {
    const dim3 grid(num_tiles, a.nsplit);
    if (key_tile == 64) {
        cudaFuncSetAttribute(talking_attention_kernel<T, TOK, VC2, 2>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        talking_attention_kernel<T, TOK, VC2, 2><<<grid, TA_WARPS * 32, smem, stream>>>(a);
    } else {
        cudaFuncSetAttribute(talking_attention_kernel<T, TOK, VC2, 1>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        talking_attention_kernel<T, TOK, VC2, 1><<<grid, TA_WARPS * 32, smem, stream>>>(a);
    }
    return FSIE_LAUNCH_CHECK();
}

template <typename T, int TOK>
int talking_attention_launch_tok(const TalkingArgs& a, int num_tiles, int key_tile, size_t smem,
                                 cudaStream_t stream) {
    const int pairs = (a.vdim + 63) / 64;
    if (pairs <= 1) return talking_attention_launch_tile<T, TOK, 1>(a, num_tiles, key_tile, smem, stream);
    if (pairs <= 2) return talking_attention_launch_tile<T, TOK, 2>(a, num_tiles, key_tile, smem, stream);
    return talking_attention_launch_tile<T, TOK, 4>(a, num_tiles, key_tile, smem, stream);
}

template <typename T>
int talking_attention_launch(TalkingArgs a, int num_tiles, cudaStream_t stream) {
    if (num_tiles <= 0) return 0;
    if (a.heads <= 0 || a.kv_heads <= 0 || a.heads % a.kv_heads || a.window < 0 || a.keep_first < 0 ||
        a.nsplit < 1 || a.nsplit > 65535 ||
        (a.tile_tokens != 1 && a.tile_tokens != 2 && a.tile_tokens != 4 && a.tile_tokens != 8) ||
        a.tile_tokens * ((a.heads + TA_WARPS - 1) / TA_WARPS) > 8)
        return ERR_BAD_ARGUMENT;
    if (a.vdim > 256) return ERR_UNSUPPORTED;
    const int key_tile = talking_key_tile(a.heads, a.kv_heads, a.dim, a.vdim, (int)sizeof(T));
    if (key_tile == 0) return ERR_UNSUPPORTED;
    const size_t smem = TalkingLayout(a.heads, a.kv_heads, a.dim, a.vdim, key_tile, (int)sizeof(T)).total;
    if (a.nsplit > 1 && (!a.part_stats || !a.part_out)) return ERR_BAD_ARGUMENT;
    const int first = a.nsplit > 1 ? 1 : 0, last = a.nsplit > 1 ? 2 : 0;
    for (int mode = first; mode <= last; ++mode) {
        a.mode = mode;
        int code;
        switch (a.tile_tokens) {
            case 1: code = talking_attention_launch_tok<T, 1>(a, num_tiles, key_tile, smem, stream); break;
            case 2: code = talking_attention_launch_tok<T, 2>(a, num_tiles, key_tile, smem, stream); break;
            case 4: code = talking_attention_launch_tok<T, 4>(a, num_tiles, key_tile, smem, stream); break;
            default: code = talking_attention_launch_tok<T, 8>(a, num_tiles, key_tile, smem, stream); break;
        }
        if (code) return code;
    }
    if (a.nsplit > 1) {
        const long long count = (long long)a.tokens * a.heads * a.vdim;
        const long long wanted = (count + 255) / 256;
        talking_attention_merge_kernel<T><<<(unsigned)(wanted > 2048 ? 2048 : wanted), 256, 0, stream>>>(
            a.part_out, reinterpret_cast<T*>(a.out), count, a.nsplit);
        return FSIE_LAUNCH_CHECK();
    }
    return 0;
}

}  // namespace fsie
