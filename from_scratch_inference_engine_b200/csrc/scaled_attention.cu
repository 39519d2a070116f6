// Causal softmax attention over the paged cache with a scale per query head, keys and values of
// different widths, and optionally values that ARE the leading columns of the key rows (a cache
// that stores one latent row per token, read by every head as key and as value).  32-bit
// arithmetic on the CUDA cores for any sizes; storage type T (float or bfloat16) for q, the pages
// and the output.
//
//   s_h(i, j) = (q_h,i . k_g(h),j) * head_scale[h]      visible: j <= i and (window == 0 or i - j < window)
//   o_h,i     = sum_j softmax_j(s_h(i, .)) v_g(h),j      g(h) = h / (heads / kv_heads)
//
// Work is cut as in attention_generic.cu: a tile is up to ROWS query rows of one request and one
// key/value head, a row being (token, head of the group): row = token * group + head_in_group; a
// tile's key range may be split over blockIdx.z and merged by sa_combine_kernel.
//
// The file also holds the step before it for projections q | k | v laid out head by head:
// rotation of q and k over the leading `rotary_dim` of each head (pairs i, i + rotary_dim / 2),
// blending of v with the values another layer computed for the same token, and the cache write.
#include "common.cuh"
#include <math.h>

namespace fsie {

constexpr int SA_ROWS = 32;
constexpr int SA_WARPS = 8;
constexpr int SA_RPW = SA_ROWS / SA_WARPS;
constexpr int SA_KT = 32;

struct ScaledAttnParams {
    const void* q; int q_ld;                  // head h of token t at t * q_ld + h * key_dim
    const float* head_scale;                  // [heads]
    const void* k_pages; const void* v_pages;
    long long page_stride; int page_size;
    int key_dim, value_dim, value_ld;         // value rows are value_ld apart (key_dim when they live in the key rows)
    const int* block_tables; int bt_stride;
    const int* tile_item; const int* tile_row0;
    const int* item_qstart; const int* item_qlen; const int* item_pos0; const int* item_slots;
    void* out; int out_ld;                    // head h of token t at t * out_ld + h * value_dim
    float* part_o; float* part_ml;            // [nsplit, tokens, heads, value_dim], [nsplit, tokens, heads, 2]
    int tokens, heads, kv_heads, window, nsplit;
    int* error;
};

template <typename T, int DPL, bool SHARED_V>
__global__ void __launch_bounds__(SA_WARPS * 32) scaled_attention_kernel(const ScaledAttnParams p) {
    extern __shared__ __align__(16) float sa_smem[];
    const int dk = p.key_dim, dv = p.value_dim;
    const int dk4 = (dk + 3) & ~3;
    float* qs = sa_smem;                              // [ROWS][dk4]
    float* ks = qs + SA_ROWS * dk4;                   // [KT][dk4 + 1]
    float* vs = ks + SA_KT * (dk4 + 1);               // [KT][dv] unless the values live in the key rows
    __shared__ long long key_base[SA_KT];
    __shared__ long long value_base[SA_KT];

    const int kvh = blockIdx.x, tile = blockIdx.y, split = blockIdx.z;
    const int group = p.heads / p.kv_heads;
    grid_dependency_wait();
    grid_dependents_go();
    const int item = p.tile_item[tile];
    if (p.item_slots && p.item_slots[item] < 0) return;      // a padding entry of a fixed-size batch
    const int row0 = p.tile_row0[tile];
    const int qstart = p.item_qstart[item], qlen = p.item_qlen[item], pos0 = p.item_pos0[item];
    const int nrows = min(SA_ROWS, qlen * group - row0);
    if (nrows <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const T* q = (const T*)p.q;
    const T* kp = (const T*)p.k_pages;
    const T* vp = (const T*)p.v_pages;
    const int* bt = p.block_tables + (size_t)item * p.bt_stride;

    // the tile's query rows, multiplied by their head's scale, zero beyond the tile and the key size
    for (int r = warp; r < SA_ROWS; r += SA_WARPS) {
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        const float sc = r < nrows ? p.head_scale[h] : 0.f;
        for (int d = lane; d < dk4; d += 32)
            qs[r * dk4 + d] = (r < nrows && d < dk) ? to_float(q[(size_t)tok * p.q_ld + (size_t)h * dk + d]) * sc : 0.f;
    }

    const int pos_first = pos0 + row0 / group;
    const int pos_last = pos0 + (row0 + nrows - 1) / group;
    int kbegin = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int kend = pos_last + 1;
    if (p.nsplit > 1) {
        const int span = kend - kbegin;
        int chunk = (span + p.nsplit - 1) / p.nsplit;
        chunk = ((chunk + SA_KT - 1) / SA_KT) * SA_KT;
        const int b = kbegin + split * chunk;
        kend = min(kend, b + chunk);
        kbegin = b;
    }

    float m[SA_RPW], l[SA_RPW], acc[SA_RPW][DPL];
    int pos[SA_RPW];
#pragma unroll
    for (int i = 0; i < SA_RPW; ++i) {
        m[i] = -INFINITY; l[i] = 0.f;
        const int r = warp * SA_RPW + i;
        pos[i] = r < nrows ? pos0 + (row0 + r) / group : -1;       // -1: no row, sees nothing
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[i][c] = 0.f;
    }

    for (int k0 = kbegin; k0 < kend; k0 += SA_KT) {
        __syncthreads();
        if (tid < SA_KT) {
            const int kj = k0 + tid;
            long long kb = -1, vb = -1;
            if (kj < kend) {
                const int page = bt[kj / p.page_size];
                if (page >= 0) {
                    const long long at = (long long)kvh * p.page_size + kj % p.page_size;
                    kb = (long long)page * p.page_stride + at * dk;
                    vb = (long long)page * p.page_stride + at * p.value_ld;
                } else if (kj <= pos_last && (p.window <= 0 || kj > pos_first - p.window) && p.error) {
                    atomicExch(p.error, 3);            // some row of the tile sees this key, and its page was given back
                }
            }
            key_base[tid] = kb;
            value_base[tid] = vb;
        }
        __syncthreads();
        for (int j = warp; j < SA_KT; j += SA_WARPS) {
            const long long kb = key_base[j];
            for (int d = lane; d < dk4; d += 32)
                ks[j * (dk4 + 1) + d] = (kb >= 0 && d < dk) ? to_float(kp[kb + d]) : 0.f;
            if (!SHARED_V) {
                const long long vb = value_base[j];
                for (int d = lane; d < dv; d += 32) vs[j * dv + d] = vb >= 0 ? to_float(vp[vb + d]) : 0.f;
            }
        }
        __syncthreads();
        if (warp * SA_RPW >= nrows) continue;          // a warp without rows (it still took part in the copies)
        const int kj = k0 + lane;
        const bool key_ok = kj < kend && key_base[lane] >= 0;
        float s[SA_RPW];
#pragma unroll
        for (int i = 0; i < SA_RPW; ++i) s[i] = 0.f;
        const float* kr = ks + lane * (dk4 + 1);
        const float* qr = qs + warp * SA_RPW * dk4;
        for (int d = 0; d < dk4; d += 4) {
            const float k0v = kr[d], k1v = kr[d + 1], k2v = kr[d + 2], k3v = kr[d + 3];
#pragma unroll
            for (int i = 0; i < SA_RPW; ++i) {
                const float4 qq = *reinterpret_cast<const float4*>(qr + i * dk4 + d);
                s[i] = fmaf(qq.x, k0v, s[i]);
                s[i] = fmaf(qq.y, k1v, s[i]);
                s[i] = fmaf(qq.z, k2v, s[i]);
                s[i] = fmaf(qq.w, k3v, s[i]);
            }
        }
        float pj[SA_RPW];
        bool any = false;
#pragma unroll
        for (int i = 0; i < SA_RPW; ++i) {
            const bool seen = key_ok && kj <= pos[i] && (p.window <= 0 || kj > pos[i] - p.window);
            const float si = seen ? s[i] : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(si));
            if (m_new == -INFINITY) { pj[i] = 0.f; continue; }       // uniform over the warp
            const float corr = expf(m[i] - m_new);
            pj[i] = seen ? expf(si - m_new) : 0.f;
            l[i] = l[i] * corr + warp_sum(pj[i]);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[i][c] *= corr;
            any = true;
        }
        if (!any) continue;
        const int nk = min(SA_KT, kend - k0);
        for (int j = 0; j < nk; ++j) {
            float pw[SA_RPW];
#pragma unroll
            for (int i = 0; i < SA_RPW; ++i) pw[i] = __shfl_sync(0xffffffffu, pj[i], j);
            const float* vr = SHARED_V ? ks + j * (dk4 + 1) : vs + j * dv;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                const float v = d < dv ? vr[d] : 0.f;
#pragma unroll
                for (int i = 0; i < SA_RPW; ++i) acc[i][c] = fmaf(pw[i], v, acc[i][c]);
            }
        }
    }

#pragma unroll
    for (int i = 0; i < SA_RPW; ++i) {
        const int r = warp * SA_RPW + i;
        if (r >= nrows) continue;
        const int row = row0 + r;
        const int tok = qstart + row / group, h = kvh * group + row % group;
        if (p.nsplit == 1) {
            T* o = (T*)p.out + (size_t)tok * p.out_ld + (size_t)h * dv;
            const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) o[d] = from_float<T>(acc[i][c] * inv);
            }
        } else {
            const size_t idx = ((size_t)split * p.tokens + tok) * p.heads + h;
            float* o = p.part_o + idx * dv;
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < dv) o[d] = acc[i][c];
            }
            if (lane == 0) { p.part_ml[idx * 2] = m[i]; p.part_ml[idx * 2 + 1] = l[i]; }
        }
    }
}

// o = sum_z acc_z e^(m_z - M) / sum_z l_z e^(m_z - M) over the key ranges z of one (token, head)
template <typename T>
__global__ void sa_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  T* __restrict__ out, int out_ld, int tokens, int heads, int dv,
                                  int nsplit) {
    const int tok = blockIdx.x, h = blockIdx.y;
    float mmax = -INFINITY;
    for (int z = 0; z < nsplit; ++z)
        mmax = fmaxf(mmax, part_ml[(((size_t)z * tokens + tok) * heads + h) * 2]);
    float denom = 0.f;
    for (int z = 0; z < nsplit; ++z) {
        const size_t idx = ((size_t)z * tokens + tok) * heads + h;
        const float mz = part_ml[idx * 2];
        if (mz != -INFINITY) denom += part_ml[idx * 2 + 1] * expf(mz - mmax);
    }
    const float inv = denom > 0.f ? 1.0f / denom : 0.f;
    for (int d = threadIdx.x; d < dv; d += blockDim.x) {
        float o = 0.f;
        for (int z = 0; z < nsplit; ++z) {
            const size_t idx = ((size_t)z * tokens + tok) * heads + h;
            const float mz = part_ml[idx * 2];
            if (mz != -INFINITY) o += part_o[idx * dv + d] * expf(mz - mmax);
        }
        out[(size_t)tok * out_ld + (size_t)h * dv + d] = from_float<T>(o * inv);
    }
}

// One block per token of proj = [ q (heads x dim) | k (kv_heads x dim) | v (kv_heads x vdim) ].
//   q, k   pairs (i, i + rotary_dim / 2) of every head turn by the token's angles (cos | sin rows of
//          the table); q in place, k into its page
//   v      mix_mode 1: also copied as it is into v_first[t];  2: v <- (1 - mix) v + mix v_first[t];
//          then into its page.  mix is one float on the device.
template <typename T>
__global__ void rotate_mix_write_kernel(T* __restrict__ proj, int ld, const int* __restrict__ positions,
                                        const float* __restrict__ cos_sin, int table_len,
                                        const int* __restrict__ slot_of, T* __restrict__ k_pages,
                                        T* __restrict__ v_pages, long long page_stride, int page_size,
                                        int heads, int kv_heads, int dim, int vdim, int rotary_dim,
                                        int mix_mode, const float* __restrict__ mix, T* __restrict__ v_first,
                                        int* __restrict__ error) {
    const int t = blockIdx.x;
    grid_dependency_wait();
    grid_dependents_go();
    const int pos = positions[t];
    if (rotary_dim > 0 && (pos < 0 || pos >= table_len)) {
        if (threadIdx.x == 0) atomicExch(error, 2);
        return;
    }
    const int half = rotary_dim / 2;
    const float* cs = cos_sin + (size_t)pos * rotary_dim;
    T* row = proj + (size_t)t * ld;
    const int slot = slot_of ? slot_of[t] : -1;
    const long long page = slot >= 0 ? slot / page_size : -1;
    const int off = slot >= 0 ? slot % page_size : 0;
    // queries: rotated in place
    for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
        const int h = e / half, i = e - h * half;
        T* a = row + h * dim + i;
        const float u = to_float(a[0]), v = to_float(a[half]);
        const float c = cs[i], s = cs[half + i];
        a[0] = from_float<T>(u * c - v * s);
        a[half] = from_float<T>(v * c + u * s);
    }
    if (slot < 0) return;
    // keys: rotated pairs and the columns that pass unchanged, into the page
    const T* k = row + heads * dim;
    for (int e = threadIdx.x; e < kv_heads * dim; e += blockDim.x) {
        const int g = e / dim, d = e - g * dim;
        float val = to_float(k[e]);
        if (d < rotary_dim) {
            const int i = d < half ? d : d - half;
            const float c = cs[i], s = cs[half + i];
            const float other = to_float(k[g * dim + (d < half ? d + half : d - half)]);
            val = d < half ? val * c - other * s : val * c + other * s;
        }
        k_pages[page * page_stride + ((long long)g * page_size + off) * dim + d] = from_float<T>(val);
    }
    // values: blended with the first blending layer's, into the page
    const T* v = k + kv_heads * dim;
    const float lambda = mix_mode == 2 ? mix[0] : 0.f;
    for (int e = threadIdx.x; e < kv_heads * vdim; e += blockDim.x) {
        const int g = e / vdim, d = e - g * vdim;
        float val = to_float(v[e]);
        if (mix_mode == 1) v_first[(size_t)t * kv_heads * vdim + e] = v[e];
        if (mix_mode == 2) val = (1.0f - lambda) * val + lambda * to_float(v_first[(size_t)t * kv_heads * vdim + e]);
        v_pages[page * page_stride + ((long long)g * page_size + off) * vdim + d] = from_float<T>(val);
    }
}

template <typename T, int DPL>
static int scaled_attention_launch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const int dk4 = (p.key_dim + 3) & ~3;
    const size_t smem = sizeof(float) * ((size_t)SA_ROWS * dk4 + (size_t)SA_KT * (dk4 + 1) +
                                         (shared_v ? 0 : (size_t)SA_KT * p.value_dim));
    if (smem > 220 * 1024) return ERR_UNSUPPORTED;
    const dim3 grid(p.kv_heads, tiles, p.nsplit);
    if (shared_v) {
        cudaFuncSetAttribute(scaled_attention_kernel<T, DPL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_dependent(scaled_attention_kernel<T, DPL, true>, grid, dim3(SA_WARPS * 32), smem, stream, p);
    }
    cudaFuncSetAttribute(scaled_attention_kernel<T, DPL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_dependent(scaled_attention_kernel<T, DPL, false>, grid, dim3(SA_WARPS * 32), smem, stream, p);
}

template <typename T>
static int scaled_attention_dispatch(const ScaledAttnParams& p, int tiles, bool shared_v, cudaStream_t stream) {
    const int dpl = (p.value_dim + 31) / 32;
    if (dpl <= 2) return scaled_attention_launch<T, 2>(p, tiles, shared_v, stream);
    if (dpl <= 4) return scaled_attention_launch<T, 4>(p, tiles, shared_v, stream);
    if (dpl <= 8) return scaled_attention_launch<T, 8>(p, tiles, shared_v, stream);
    if (dpl <= 16) return scaled_attention_launch<T, 16>(p, tiles, shared_v, stream);
    return ERR_UNSUPPORTED;
}

}  // namespace fsie

using namespace fsie;

extern "C" {

int fsie_scaled_attention_rows() { return SA_ROWS; }

// values_in_keys != 0: v_pages is ignored, a key row's first value_dim columns are its value row.
// With nsplit > 1 the caller gives part_o [nsplit, tokens, heads, value_dim] and part_ml
// [nsplit, tokens, heads, 2] (float); the ranges are merged after the launch.
int fsie_scaled_attention(const void* q, int q_ld, const float* head_scale, const void* k_pages,
                          const void* v_pages, long long page_stride, int page_size, int key_dim,
                          int value_dim, int values_in_keys, const int* block_tables, int bt_stride,
                          const int* tile_item, const int* tile_row0, int tiles, const int* item_qstart,
                          const int* item_qlen, const int* item_pos0, const int* item_slots, void* out,
                          int out_ld, float* part_o, float* part_ml, int tokens, int heads, int kv_heads,
                          int window, int nsplit, int dtype, int* error, cudaStream_t stream) {
    if (tokens <= 0 || tiles <= 0) return 0;
    if (tiles > 65535 || nsplit > 65535) return ERR_UNSUPPORTED;
    if (key_dim <= 0 || value_dim <= 0 || kv_heads <= 0 || heads % kv_heads != 0 || nsplit < 1 ||
        page_size <= 0 || window < 0 || (values_in_keys && value_dim > key_dim))
        return ERR_BAD_ARGUMENT;
    if (nsplit > 1 && (!part_o || !part_ml)) return ERR_BAD_ARGUMENT;
    ScaledAttnParams p;
    p.q = q; p.q_ld = q_ld; p.head_scale = head_scale;
    p.k_pages = k_pages; p.v_pages = values_in_keys ? k_pages : v_pages;
    p.page_stride = page_stride; p.page_size = page_size;
    p.key_dim = key_dim; p.value_dim = value_dim; p.value_ld = values_in_keys ? key_dim : value_dim;
    p.block_tables = block_tables; p.bt_stride = bt_stride;
    p.tile_item = tile_item; p.tile_row0 = tile_row0;
    p.item_qstart = item_qstart; p.item_qlen = item_qlen; p.item_pos0 = item_pos0; p.item_slots = item_slots;
    p.out = out; p.out_ld = out_ld; p.part_o = part_o; p.part_ml = part_ml;
    p.tokens = tokens; p.heads = heads; p.kv_heads = kv_heads; p.window = window; p.nsplit = nsplit;
    p.error = error;
    int rc = dtype == DTYPE_F32 ? scaled_attention_dispatch<float>(p, tiles, values_in_keys != 0, stream)
                                : scaled_attention_dispatch<bf16>(p, tiles, values_in_keys != 0, stream);
    if (rc != 0 || nsplit == 1) return rc;
    const dim3 cgrid(tokens, heads);
    const int threads = value_dim >= 128 ? 128 : (value_dim >= 64 ? 64 : 32);
    if (dtype == DTYPE_F32)
        sa_combine_kernel<float><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (float*)out, out_ld, tokens, heads, value_dim, nsplit);
    else
        sa_combine_kernel<bf16><<<cgrid, threads, 0, stream>>>(part_o, part_ml, (bf16*)out, out_ld, tokens, heads, value_dim, nsplit);
    return FSIE_LAUNCH_CHECK();
}

// proj [tokens, ld] = q | k | v head by head; cos_sin [table_len, rotary_dim]; slot_of [tokens]
// (page * page_size + offset, -1: store nothing).  mix_mode 0: values as they are; 1: values also
// copied to v_first [tokens, kv_heads * vdim]; 2: values blended with v_first by *mix.
int fsie_rotate_mix_write(void* proj, int ld, const int* positions, const float* cos_sin, int table_len,
                          const int* slot_of, void* k_pages, void* v_pages, long long page_stride,
                          int page_size, int tokens, int heads, int kv_heads, int dim, int vdim,
                          int rotary_dim, int mix_mode, const float* mix, void* v_first, int dtype,
                          int* error, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > dim || (rotary_dim & 1) || mix_mode < 0 || mix_mode > 2 ||
        (mix_mode != 0 && !v_first) || (mix_mode == 2 && !mix) || ld < (heads + kv_heads) * dim + kv_heads * vdim)
        return ERR_BAD_ARGUMENT;
    if (dtype == DTYPE_F32)
        return launch_dependent(rotate_mix_write_kernel<float>, dim3(tokens), dim3(256), 0, stream,
                                (float*)proj, ld, positions, cos_sin, table_len, slot_of, (float*)k_pages,
                                (float*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim,
                                rotary_dim, mix_mode, mix, (float*)v_first, error);
    return launch_dependent(rotate_mix_write_kernel<bf16>, dim3(tokens), dim3(256), 0, stream,
                            (bf16*)proj, ld, positions, cos_sin, table_len, slot_of, (bf16*)k_pages,
                            (bf16*)v_pages, page_stride, page_size, heads, kv_heads, dim, vdim,
                            rotary_dim, mix_mode, mix, (bf16*)v_first, error);
}

}  // extern "C"
