// Attention whose weights are sigmoids of the biased scores, over the paged cache.
//
// For a query at position p of head h (kv head h / group) and the keys j with
// 0 <= p - j < window (all j <= p without a window):
//     out = sum_j sigmoid((q . K_j) * scale + bias[h]) V_j
// Nothing is normalised over the keys, so there is no running maximum and no
// denominator, and partial sums over any split of the keys simply add.  Keys are
// `head_dim` wide, values `v_dim` (the two page tensors have their own widths).
//
// sig_qkv_post: the rows of a stacked product [q | k | v] (32-bit or bfloat16,
// the first columns of a possibly wider row): the first `rot_dims` dimensions of
// every q and k head turn in half-split pairs (i with i + rot_dims / 2) by the
// angle position / denom[i]; q goes out [R, nq * head_dim], k and v into their
// pages at the row's position.  All arithmetic is 32-bit; sine and cosine come
// from `exact_sincosf`.
//
// attention_sigmoid_plain: one warp per (query row, head), keys one after another:
// the 32-bit path, any head sizes up to 512, and the form the tensor-core kernels
// are compared with.  attention_sigmoid_mma: bfloat16, mma.sync m16n8k16, a warp
// takes 16 rows of (position, head of one kv group) against a page of keys at a
// time (prompts and decode rows alike; a decode row's 16 rows are its group's
// heads).
#include "common.cuh"
#include "exact_math.cuh"
#include "paged.cuh"

namespace {

using namespace rfx;

constexpr int MAX_PER_LANE = 16;  // head sizes up to 512 in the plain kernel

__device__ __forceinline__ size_t page_offset(const int* page_table, int max_pages, int page_size, int nkv,
                                              int slot, int pos, int kvh, int width) {
    const int page = page_table[(size_t)slot * max_pages + pos / page_size];
    return (((size_t)page * nkv + kvh) * page_size + (pos % page_size)) * (size_t)width;
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
sig_qkv_post_kernel(const TI* __restrict__ proj, int ldp, int col0, const float* __restrict__ denom, int rot_dims,
                    const int* __restrict__ row_pos, const int* __restrict__ row_slot, TO* __restrict__ q_out,
                    TO* __restrict__ k_pages, TO* __restrict__ v_pages, const int* __restrict__ page_table,
                    int max_pages, int page_size, int nq, int nkv, int d, int dv, int writes_cache) {
    extern __shared__ float cs[];  // [rot_dims / 2] cosines, then as many sines
    pdl_prologue();
    const int r = blockIdx.x;
    const int pos = row_pos[r], slot = row_slot[r];
    const int half = rot_dims / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float s, c;
        exact_sincosf((float)pos / denom[i], &s, &c);
        cs[i] = c;
        cs[half + i] = s;
    }
    __syncthreads();
    const TI* row = proj + (size_t)r * ldp + col0;
    const int n_qk = (nq + (writes_cache ? nkv : 0)) * d;
    for (int e = threadIdx.x; e < n_qk; e += blockDim.x) {
        const int head = e / d, i = e - head * d;
        float v = ld<TI>(row, e);
        if (i < rot_dims) {
            const int f = i < half ? i : i - half;
            const float partner = ld<TI>(row, i < half ? e + half : e - half);
            // (u, v) -> (u cos - v sin, v cos + u sin)
            v = fmaf(partner, i < half ? -cs[half + f] : cs[half + f], __fmul_rn(v, cs[f]));
        }
        if (head < nq) {
            st<TO>(q_out, (size_t)r * nq * d + e, v);
        } else {
            const size_t off = page_offset(page_table, max_pages, page_size, nkv, slot, pos, head - nq, d);
            st<TO>(k_pages, off + i, v);
        }
    }
    if (!writes_cache) return;
    const TI* vrow = row + (size_t)(nq + nkv) * d;
    for (int e = threadIdx.x; e < nkv * dv; e += blockDim.x) {
        const int head = e / dv, i = e - head * dv;
        const size_t off = page_offset(page_table, max_pages, page_size, nkv, slot, pos, head, dv);
        st<TO>(v_pages, off + i, ld<TI>(vrow, e));
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
attention_sigmoid_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                               const int* __restrict__ page_table, int max_pages, int page_size,
                               const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                               T* __restrict__ out, int nq, int nkv, int d, int dv, int window, float scale,
                               const float* __restrict__ bias) {
    pdl_prologue();
    const int r = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * (blockDim.x >> 5) + warp;
    if (h >= nq) return;
    const int kvh = h / (nq / nkv);
    const int pos = row_pos[r], slot = row_slot[r];
    const int lo = (window > 0 && pos + 1 > window) ? pos + 1 - window : 0;
    float qv[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = q + ((size_t)r * nq + h) * d;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        qv[i] = e < d ? ld<T>(qrow, e) : 0.0f;
        acc[i] = 0.0f;
    }
    const float b = bias ? bias[h] : 0.0f;
    for (int j = lo; j <= pos; ++j) {
        const T* kp = k_pages + page_offset(page_table, max_pages, page_size, nkv, slot, j, kvh, d);
        const T* vp = v_pages + page_offset(page_table, max_pages, page_size, nkv, slot, j, kvh, dv);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (e < d) dot = fmaf(qv[i], ld<T>(kp, e), dot);
        }
        const float s = fmaf(warp_sum(dot), scale, b);
        const float p = 1.0f / (1.0f + exact_expf(-s));
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (e < dv) acc[i] = fmaf(p, ld<T>(vp, e), acc[i]);
        }
    }
    T* orow = out + ((size_t)r * nq + h) * dv;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        if (e < dv) st<T>(orow, e, acc[i]);
    }
}

}  // namespace

extern "C" int rfx_sig_qkv_post(const void* proj, int in_dt, int ld, int col0, const float* denom, int rot_dims,
                                const int* row_pos, const int* row_slot, void* q_out, void* k_pages, void* v_pages,
                                int out_dt, const int* page_table, int max_pages, int page_size, int R, int nq,
                                int nkv, int d, int dv, int writes_cache, void* stream) {
    if (R <= 0) return 0;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > d) return RFX_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)rot_dims * sizeof(float);
#define RFX_GO(TI, TO)                                                                                        \
    RFX_LAUNCH((sig_qkv_post_kernel<TI, TO>), R, 256, smem, s, (const TI*)proj, ld, col0, denom, rot_dims,   \
               row_pos, row_slot, (TO*)q_out, (TO*)k_pages, (TO*)v_pages, page_table, max_pages, page_size,   \
               nq, nkv, d, dv, writes_cache)
    if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_F32) RFX_GO(float, float);
    else if (in_dt == RFX_DT_F32 && out_dt == RFX_DT_BF16) RFX_GO(float, __nv_bfloat16);
    else if (in_dt == RFX_DT_BF16 && out_dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16, __nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_attention_sigmoid_plain(const void* q, const void* k_pages, const void* v_pages, int dt,
                                           const int* page_table, int max_pages, int page_size, const int* row_pos,
                                           const int* row_slot, void* out, int R, int nq, int nkv, int d, int dv,
                                           int window, float scale, const float* bias, void* stream) {
    if (R <= 0) return 0;
    if (d <= 0 || dv <= 0 || d > 32 * MAX_PER_LANE || dv > 32 * MAX_PER_LANE) return RFX_ERR_UNSUPPORTED;
    if (nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    dim3 grid(R, (nq + 3) / 4);
    if (grid.y > 65535) return RFX_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(attention_sigmoid_plain_kernel<float>, grid, 128, 0, s, (const float*)q, (const float*)k_pages,
                   (const float*)v_pages, page_table, max_pages, page_size, row_pos, row_slot, (float*)out, nq, nkv,
                   d, dv, window, scale, bias);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(attention_sigmoid_plain_kernel<__nv_bfloat16>, grid, 128, 0, s, (const __nv_bfloat16*)q,
                   (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, page_table, max_pages, page_size,
                   row_pos, row_slot, (__nv_bfloat16*)out, nq, nkv, d, dv, window, scale, bias);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}
