// The mixed-heads window attention for prompt portions on the tensor cores (bfloat16 pages).
//
// The mixing is moved to the output side: with a_(h',c) = softmax_h' applied to the values of
// key/value head c,
//     o_h = sum_h' talk[h, h'] a_(h', g(h))
// so every (query head, value head) pair is an ordinary one-walk attention with a running maximum,
// and no block has to see another head's weights.  A block takes 16 consecutive tokens of one
// request and one query head; its warps share the scores against the head's keys (mma.sync
// m16n8k16, bf16 operands, float accumulators; each warp a slice of the keys) and the running
// softmax in 32-bit, and warp c applies the weights to the values of key/value head c.  The weights enter that product as the sum of two
// bfloat16 halves (p = hi + lo, two products), which keeps 16 bits of them.  A second kernel
// mixes the normalised partial outputs [token][head][value head][vdim] (float) into the output.
#include "common.cuh"

namespace fsie {

constexpr int TM_KEYS = 32;        // keys of one tile
constexpr int TM_ROWS = 16;        // tokens of one block

struct TalkingMmaArgs {
    const float* q; const bf16* k_pages; const bf16* v_pages; long long page_stride; int page_size;
    const int* block_tables; int table_stride; const int* tile_item; const int* tile_row0;
    const int* item_qstart; const int* item_qlen; const int* item_pos0; const int* item_slots;
    float* partial; int heads, kv_heads, window, keep_first; float scale; int* error;
};

__device__ __forceinline__ unsigned tm_smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void tm_ldmatrix_x2_trans(unsigned& r0, unsigned& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                 : "=r"(r0), "=r"(r1) : "r"(tm_smem_u32(p)));
}
// d += a (16 x 16, row) * b (16 x 8, col), bf16 operands, float accumulators
__device__ __forceinline__ void tm_mma(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// two floats as the high bfloat16 halves and what they leave
__device__ __forceinline__ void tm_split(float x, float y, unsigned& hi, unsigned& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 back = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - back.x, y - back.y);
    hi = *reinterpret_cast<const unsigned*>(&h);
    lo = *reinterpret_cast<const unsigned*>(&l);
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(256, 2) talking_attention_mma_kernel(const TalkingMmaArgs a) {
    constexpr int QLD = DIM + 8, VLD = VDIM + 8, PLD = TM_KEYS + 8, NT = TM_KEYS / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int H = a.heads, G = a.kv_heads;
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);             // [16][QLD]
    bf16* Ks = Qs + TM_ROWS * QLD;                            // [keys][QLD]
    bf16* Vs = Ks + TM_KEYS * QLD;                            // [G][keys][VLD]
    bf16* Ph = Vs + (size_t)G * TM_KEYS * VLD;                // [16][PLD]: the weights' high halves
    bf16* Pl = Ph + TM_ROWS * PLD;                            // ... and what the high halves leave
    float* shared_max = reinterpret_cast<float*>(Pl + TM_ROWS * PLD);   // [8 warps][16 rows]
    int* key_page = reinterpret_cast<int*>(shared_max + 8 * TM_ROWS);
    int* key_off = key_page + TM_KEYS;

    const int tile = blockIdx.x, h = blockIdx.y, kvh = h / (H / G);
    const int item = a.tile_item[tile], tok0 = a.tile_row0[tile];
    if (a.item_slots[item] < 0) return;                       // a padding entry of a fixed-size batch
    const int n_tok = min(TM_ROWS, a.item_qlen[item] - tok0);
    if (n_tok <= 0) return;
    const int p_first = a.item_pos0[item] + tok0, p_last = p_first + n_tok - 1;
    const int lo = a.window > 0 ? max(0, p_first - a.window + 1) : 0;
    const int kept = min(a.keep_first, lo);
    const int n_keys = kept + (p_last - lo + 1);
    const int token0 = a.item_qstart[item] + tok0;
    const int* table = a.block_tables + (size_t)item * a.table_stride;
    const int lane = threadIdx.x & 31, c = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;

    for (int idx = threadIdx.x; idx < TM_ROWS * DIM; idx += blockDim.x) {
        const int r = idx / DIM, d = idx - r * DIM;
        Qs[r * QLD + d] = __float2bfloat16_rn(r < n_tok ? a.q[((size_t)(token0 + r) * H + h) * DIM + d] : 0.f);
    }
    __syncthreads();
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.f, 0.f};
    float acc[VDIM / 8][4];
#pragma unroll
    for (int nt = 0; nt < VDIM / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    for (int u0 = 0; u0 < n_keys; u0 += TM_KEYS) {
        const int n = min(TM_KEYS, n_keys - u0);
        __syncthreads();                                       // the tile before is done with Ks, Vs
        if (threadIdx.x < TM_KEYS) {
            int page = -1, off = 0;
            if ((int)threadIdx.x < n) {
                const int u = u0 + threadIdx.x;
                const int j = u < kept ? u : lo + (u - kept);
                page = table[j / a.page_size];
                off = j - (j / a.page_size) * a.page_size;
                if (page < 0) atomicExch(a.error, 3);          // a visible key's page was given back
            }
            key_page[threadIdx.x] = page;
            key_off[threadIdx.x] = off;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < TM_KEYS * (DIM / 8); idx += blockDim.x) {
            const int jj = idx / (DIM / 8), ch = idx - jj * (DIM / 8);
            const int page = key_page[jj];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (page >= 0)
                v = *reinterpret_cast<const uint4*>(a.k_pages + page * a.page_stride +
                        ((size_t)kvh * a.page_size + key_off[jj]) * DIM + ch * 8);
            *reinterpret_cast<uint4*>(Ks + jj * QLD + ch * 8) = v;
        }
        for (int idx = threadIdx.x; idx < G * TM_KEYS * (VDIM / 8); idx += blockDim.x) {
            const int ch = idx % (VDIM / 8), jj = (idx / (VDIM / 8)) % TM_KEYS, gv = idx / ((VDIM / 8) * TM_KEYS);
            const int page = key_page[jj];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (page >= 0)
                v = *reinterpret_cast<const uint4*>(a.v_pages + page * a.page_stride +
                        ((size_t)gv * a.page_size + key_off[jj]) * VDIM + ch * 8);
            *reinterpret_cast<uint4*>(Vs + ((size_t)gv * TM_KEYS + jj) * VLD + ch * 8) = v;
        }
        __syncthreads();

        // The scores of the tile are computed once per block: warp c takes the 8-key slices c,
        // c + G, ...; the slices' maxima and the weights (as two bfloat16 halves) meet in shared
        // memory, from where every warp reads all of them for its own value head.
        float s[NT][4];
#pragma unroll
        for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < DIM / 16; ++ks) {
            // the q fragment of this step (the tile stays in shared memory: keeping all steps'
            // fragments in registers would halve the blocks an SM holds)
            const bf16* base = Qs + ks * 16 + 2 * t;
            const unsigned qa[4] = {*reinterpret_cast<const unsigned*>(base + g * QLD),
                                    *reinterpret_cast<const unsigned*>(base + (g + 8) * QLD),
                                    *reinterpret_cast<const unsigned*>(base + g * QLD + 8),
                                    *reinterpret_cast<const unsigned*>(base + (g + 8) * QLD + 8)};
#pragma unroll
            for (int i = 0; i < NT; ++i) {
                const int nt = c + i * G;
                if (nt >= NT) break;
                const bf16* kb = Ks + (nt * 8 + g) * QLD + ks * 16 + 2 * t;
                tm_mma(s[i], qa, *reinterpret_cast<const unsigned*>(kb),
                       *reinterpret_cast<const unsigned*>(kb + 8));
            }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int nt = c + i * G;
            if (nt >= NT) break;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = e >> 1, tok = g + 8 * row, key = nt * 8 + 2 * t + (e & 1);
                const int u = u0 + key;
                const int j = u < kept ? u : lo + (u - kept);
                const int p_i = p_first + tok;
                const bool see = key < n && tok < n_tok && j <= p_i &&
                    (a.window <= 0 || p_i - j < a.window || j < a.keep_first);
                s[i][e] = see ? s[i][e] * a.scale : -INFINITY;
                tile_max[row] = fmaxf(tile_max[row], s[i][e]);
            }
        }
#pragma unroll
        for (int row = 0; row < 2; ++row) {
            tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 1));
            tile_max[row] = fmaxf(tile_max[row], __shfl_xor_sync(0xffffffffu, tile_max[row], 2));
            if (t == 0) shared_max[c * TM_ROWS + g + 8 * row] = tile_max[row];
        }
        __syncthreads();
#pragma unroll
        for (int row = 0; row < 2; ++row) {
            float all = -INFINITY;
            for (int w = 0; w < G; ++w) all = fmaxf(all, shared_max[w * TM_ROWS + g + 8 * row]);
            const float m_new = fmaxf(row_max[row], all);
            const float alpha = m_new == -INFINITY ? 1.f : expf(row_max[row] - m_new);
            row_max[row] = m_new;
            row_sum[row] *= alpha;
#pragma unroll
            for (int nt = 0; nt < VDIM / 8; ++nt) {
                acc[nt][2 * row] *= alpha;
                acc[nt][2 * row + 1] *= alpha;
            }
        }
#pragma unroll
        for (int i = 0; i < NT; ++i) {
            const int nt = c + i * G;
            if (nt >= NT) break;
            float p[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                p[e] = s[i][e] == -INFINITY ? 0.f : expf(s[i][e] - row_max[e >> 1]);
                row_sum[e >> 1] += p[e];
            }
            unsigned hi, low;
            tm_split(p[0], p[1], hi, low);
            *reinterpret_cast<unsigned*>(Ph + g * PLD + nt * 8 + 2 * t) = hi;
            *reinterpret_cast<unsigned*>(Pl + g * PLD + nt * 8 + 2 * t) = low;
            tm_split(p[2], p[3], hi, low);
            *reinterpret_cast<unsigned*>(Ph + (g + 8) * PLD + nt * 8 + 2 * t) = hi;
            *reinterpret_cast<unsigned*>(Pl + (g + 8) * PLD + nt * 8 + 2 * t) = low;
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < TM_KEYS / 16; ++ks) {
            const bf16* ph = Ph + g * PLD + ks * 16 + 2 * t;
            const bf16* pl = Pl + g * PLD + ks * 16 + 2 * t;
            const unsigned hi[4] = {*reinterpret_cast<const unsigned*>(ph),
                                    *reinterpret_cast<const unsigned*>(ph + 8 * PLD),
                                    *reinterpret_cast<const unsigned*>(ph + 8),
                                    *reinterpret_cast<const unsigned*>(ph + 8 * PLD + 8)};
            const unsigned lo2[4] = {*reinterpret_cast<const unsigned*>(pl),
                                     *reinterpret_cast<const unsigned*>(pl + 8 * PLD),
                                     *reinterpret_cast<const unsigned*>(pl + 8),
                                     *reinterpret_cast<const unsigned*>(pl + 8 * PLD + 8)};
            const bf16* vrow = Vs + ((size_t)c * TM_KEYS + ks * 16 + (lane & 15)) * VLD;
#pragma unroll
            for (int nt = 0; nt < VDIM / 8; ++nt) {
                unsigned b0, b1;
                tm_ldmatrix_x2_trans(b0, b1, vrow + nt * 8);
                tm_mma(acc[nt], hi, b0, b1);
                tm_mma(acc[nt], lo2, b0, b1);
            }
        }
    }
    // every warp has summed the weights of its own key slices: the rows' sums over all of them
    __syncthreads();
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        row_sum[row] += __shfl_xor_sync(0xffffffffu, row_sum[row], 1);
        row_sum[row] += __shfl_xor_sync(0xffffffffu, row_sum[row], 2);
        if (t == 0) shared_max[c * TM_ROWS + g + 8 * row] = row_sum[row];
    }
    __syncthreads();
#pragma unroll
    for (int row = 0; row < 2; ++row) {
        float total = 0.f;
        for (int w = 0; w < G; ++w) total += shared_max[w * TM_ROWS + g + 8 * row];
        const int tok = g + 8 * row;
        if (tok >= n_tok) continue;
        const float inv = total > 0.f ? 1.0f / total : 0.f;
        float* dst = a.partial + (((size_t)(token0 + tok) * H + h) * G + c) * VDIM;
#pragma unroll
        for (int nt = 0; nt < VDIM / 8; ++nt)
            *reinterpret_cast<float2*>(dst + nt * 8 + 2 * t) =
                make_float2(acc[nt][2 * row] * inv, acc[nt][2 * row + 1] * inv);
    }
}

// out[t][h][:] = sum_h' talk[h, h'] partial[t][h'][g(h)][:]
__global__ void talking_attention_mix_kernel(const float* __restrict__ partial, const float* __restrict__ talk,
                                             bf16* __restrict__ out, long long count, int heads,
                                             int kv_heads, int vdim) {
    const int group = heads / kv_heads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (long long)gridDim.x * blockDim.x) {
        const int col = (int)(i % vdim), h = (int)((i / vdim) % heads);
        const long long tok = i / ((long long)vdim * heads);
        const float* from = partial + ((size_t)tok * heads * kv_heads + h / group) * vdim + col;
        const float* mix = talk + (size_t)h * heads;
        float v = 0.f;
        for (int h2 = 0; h2 < heads; ++h2) v += mix[h2] * from[(size_t)h2 * kv_heads * vdim];
        out[i] = __float2bfloat16_rn(v);
    }
}

}  // namespace fsie

using namespace fsie;

extern "C" {

// Whether the tensor-core form takes these sizes (1) or not (0).
int fsie_talking_attention_mma_takes(int heads, int kv_heads, int dim, int vdim) {
    if (heads <= 0 || kv_heads <= 0 || kv_heads > 8 || heads % kv_heads || heads > 65535) return 0;
    return (dim == 64 && vdim == 64) || (dim == 128 && vdim == 128);
}

// Tiles are 16 consecutive tokens of a request.  partial: float [tokens * heads * kv_heads * vdim].
int fsie_talking_attention_mma(const float* q, const void* k_pages, const void* v_pages,
                               long long page_stride, int page_size, const int* block_tables,
                               int table_stride, const int* tile_item, const int* tile_row0, int num_tiles,
                               const int* item_qstart, const int* item_qlen, const int* item_pos0,
                               const int* item_slots, const float* talk, float* partial, void* out,
                               int tokens, int heads, int kv_heads, int dim, int vdim, int window,
                               int keep_first, float scale, int* error, cudaStream_t stream) {
    if (num_tiles <= 0 || tokens <= 0) return 0;
    if (!fsie_talking_attention_mma_takes(heads, kv_heads, dim, vdim)) return ERR_UNSUPPORTED;
    if (page_stride % 8 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) || window < 0 || keep_first < 0)
        return ERR_BAD_ARGUMENT;
    TalkingMmaArgs a = {q, (const bf16*)k_pages, (const bf16*)v_pages, page_stride, page_size, block_tables,
                        table_stride, tile_item, tile_row0, item_qstart, item_qlen, item_pos0, item_slots,
                        partial, heads, kv_heads, window, keep_first, scale, error};
    const dim3 grid(num_tiles, heads);
    const int threads = 32 * kv_heads;
#define FSIE_TM(DIM, VDIM)                                                                          \
    do {                                                                                            \
        const size_t smem = ((size_t)(TM_ROWS + TM_KEYS) * (DIM + 8) +                              \
                             (size_t)kv_heads * TM_KEYS * (VDIM + 8) +                              \
                             2 * (size_t)TM_ROWS * (TM_KEYS + 8)) * sizeof(bf16) +                  \
                            8 * TM_ROWS * sizeof(float) + 2 * TM_KEYS * sizeof(int);                \
        cudaFuncSetAttribute(talking_attention_mma_kernel<DIM, VDIM>,                               \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);              \
        talking_attention_mma_kernel<DIM, VDIM><<<grid, threads, smem, stream>>>(a);                \
    } while (0)
    if (dim == 64) FSIE_TM(64, 64);
    else FSIE_TM(128, 128);
#undef FSIE_TM
    int code = FSIE_LAUNCH_CHECK();
    if (code) return code;
    const long long count = (long long)tokens * heads * vdim;
    const long long wanted = (count + 255) / 256;
    talking_attention_mix_kernel<<<(unsigned)(wanted > 4096 ? 4096 : wanted), 256, 0, stream>>>(
        partial, talk, (bf16*)out, count, heads, kv_heads, vdim);
    return FSIE_LAUNCH_CHECK();
}

}  // extern "C"
