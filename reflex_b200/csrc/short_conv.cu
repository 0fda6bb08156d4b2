// Short causal convolutions over time, one filter a channel, across steps.
//
//   y_t[c] = sum_{j < taps} w[c][j] * u_(t - taps + 1 + j)[c]      (+ cbias[c])
// with u_t = proj_t + bias, zeros before a sequence's start, the last tap on
// the current token.  The last taps - 1 inputs of every sequence are its state
// ([slot][taps - 1][channels], 32-bit, oldest first, zero when a slot is
// taken), so a step continues where the one before ended, however the tokens
// were cut.  All arithmetic is 32-bit; the taps are summed oldest first.  The
// filters come transposed, [taps][channels], so that neighbouring channels'
// taps are neighbours in memory.  Where every size is a multiple of four a
// thread takes four neighbouring channels with 16-byte accesses.
//
//  * rfx_short_conv: the convolution of a block of columns of `proj`, 32-bit out.
//  * rfx_conv_qkv_post: the convolution of the stacked q | k | v columns, then
//    what an attention needs before it can run: q times a temperature that
//    grows with the logarithm of the position,
//        1 + coef * ln(floor((p + 1) / every) + 1),
//    written head by head, and k and v into the paged cache at the row's
//    position.  Heads are stored `pad` wide (>= the key and the value size,
//    zeros beyond them), so keys and values of different sizes share one
//    attention kernel.
//  * rfx_conv_state_update: after the rows have been read, the sequences' new
//    last taps - 1 inputs.  In a step of one row a sequence rfx_short_conv_act
//    does this itself (`update`): the thread that read a channel's last inputs
//    is then their only reader.
//
// A row finds its predecessors without a map from rows to sequences: the rows
// of a sequence are neighbours, so row r - j belongs to it exactly when it has
// the same slot; what lies before the step's first row comes from the state.
#include "common.cuh"
#include "paged.cuh"

namespace {

using namespace rfx;

constexpr int MAX_TAPS = 16;

// rows of this step that precede row r in its sequence, up to `cap`; the slots of
// the rows before are loaded side by side, not one after the other's answer
__device__ __forceinline__ int rows_before(const int* __restrict__ row_slot, int r, int cap) {
    const int slot = row_slot[r];
    int t = cap;  // the nearest row back that is not this sequence's ends the count (no early exit: no chain)
    for (int j = cap - 1; j >= 0; --j) {
        const bool same = r - j - 1 >= 0 && row_slot[r - j - 1] == slot;
        if (!same) t = j;
    }
    return t;
}

// the convolution of channel c (column col0 + c of proj) at row r
__device__ __forceinline__ float conv_at(const float* __restrict__ proj, int ld, int col0, int c,
                                         const float* __restrict__ bias, const float* __restrict__ w,
                                         int taps, const float* __restrict__ state_slot, int C, int r,
                                         int before) {
    const int T = taps - 1;
    const float b = bias ? bias[c] : 0.0f;
    float y = 0.0f;
    for (int j = 0; j < taps; ++j) {
        const int back = T - j;  // tap j meets the input `back` tokens ago
        float u;
        if (back <= before) u = proj[(size_t)(r - back) * ld + col0 + c] + b;
        else u = state_slot[(size_t)(T + before - back) * C + c];
        y = fmaf(w[(size_t)j * C + c], u, y);
    }
    return y;
}

// the same for channels c .. c + 3 (every offset a multiple of four floats)
__device__ __forceinline__ float4 conv4_at(const float* __restrict__ proj, int ld, int col0, int c,
                                           const float* __restrict__ bias, const float* __restrict__ w,
                                           int taps, const float* __restrict__ state_slot, int C, int r,
                                           int before) {
    const int T = taps - 1;
    const float4 b = bias ? *reinterpret_cast<const float4*>(bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int j = 0; j < taps; ++j) {
        const int back = T - j;
        float4 u;
        if (back <= before) {
            u = *reinterpret_cast<const float4*>(proj + (size_t)(r - back) * ld + col0 + c);
            u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
        } else {
            u = *reinterpret_cast<const float4*>(state_slot + (size_t)(T + before - back) * C + c);
        }
        const float4 f = *reinterpret_cast<const float4*>(w + (size_t)j * C + c);
        y.x = fmaf(f.x, u.x, y.x);
        y.y = fmaf(f.y, u.y, y.y);
        y.z = fmaf(f.z, u.z, y.z);
        y.w = fmaf(f.w, u.w, y.w);
    }
    return y;
}

// y / (1 + e^-y), 32-bit
__device__ __forceinline__ float silu_of(float y) { return y / (1.0f + expf(-y)); }

__global__ void __launch_bounds__(256)
short_conv_kernel(const float* __restrict__ proj, int ld, int col0, const float* __restrict__ bias,
                  const float* __restrict__ w, const float* __restrict__ cbias, int taps,
                  float* state, size_t slot_stride, const int* __restrict__ row_slot,
                  float* __restrict__ out, __nv_bfloat16* __restrict__ out_lo, int C, int by4, int act,
                  int update) {
    pdl_prologue();
    const int r = blockIdx.x;
    const int before = rows_before(row_slot, r, taps - 1);
    const float* tail = state ? state + (size_t)row_slot[r] * slot_stride : nullptr;
    // `update`: every sequence has one row in this step, so the thread that read a channel's
    // last inputs is their only reader and moves them on by one (no second launch)
    float* tail_w = (update && taps > 1 && state) ? state + (size_t)row_slot[r] * slot_stride : nullptr;
    const int T = taps - 1;
    if (by4) {
        for (int c = 4 * (blockIdx.y * blockDim.x + threadIdx.x); c < C; c += 4 * gridDim.y * blockDim.x) {
            float4 y = conv4_at(proj, ld, col0, c, bias, w, taps, tail, C, r, before);
            if (cbias) {
                const float4 cb = *reinterpret_cast<const float4*>(cbias + c);
                y.x += cb.x; y.y += cb.y; y.z += cb.z; y.w += cb.w;
            }
            if (act == 1) { y.x = silu_of(y.x); y.y = silu_of(y.y); y.z = silu_of(y.z); y.w = silu_of(y.w); }
            store4(out + (size_t)r * C + c, y);
            if (out_lo) store4(out_lo + (size_t)r * C + c, y);
            if (tail_w) {
                for (int i = 0; i + 1 < T; ++i)
                    store4(tail_w + (size_t)i * C + c, *reinterpret_cast<const float4*>(tail_w + (size_t)(i + 1) * C + c));
                float4 u = *reinterpret_cast<const float4*>(proj + (size_t)r * ld + col0 + c);
                if (bias) {
                    const float4 b = *reinterpret_cast<const float4*>(bias + c);
                    u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
                }
                store4(tail_w + (size_t)(T - 1) * C + c, u);
            }
        }
        return;
    }
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        float y = conv_at(proj, ld, col0, c, bias, w, taps, tail, C, r, before) + (cbias ? cbias[c] : 0.0f);
        if (act == 1) y = silu_of(y);
        out[(size_t)r * C + c] = y;
        if (out_lo) out_lo[(size_t)r * C + c] = __float2bfloat16_rn(y);
        if (tail_w) {
            for (int i = 0; i + 1 < T; ++i) tail_w[(size_t)i * C + c] = tail_w[(size_t)(i + 1) * C + c];
            tail_w[(size_t)(T - 1) * C + c] = proj[(size_t)r * ld + col0 + c] + (bias ? bias[c] : 0.0f);
        }
    }
}

template <typename TO>
__global__ void __launch_bounds__(256)
conv_qkv_post_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias,
                     const float* __restrict__ w, int taps, const float* __restrict__ state,
                     size_t slot_stride, const int* __restrict__ row_pos, const int* __restrict__ row_slot,
                     TO* __restrict__ q_out, TO* __restrict__ k_pages, TO* __restrict__ v_pages,
                     PagedKV cache, int nq, int nkv, int dim, int vdim, int pad, float temp_coef,
                     int temp_every, int writes_cache, int by4) {
    pdl_prologue();
    const int r = blockIdx.x;
    const int pos = row_pos[r], slot = row_slot[r];
    const int before = rows_before(row_slot, r, taps - 1);
    const float* tail = state ? state + (size_t)slot * slot_stride : nullptr;
    const int C = nq * dim + nkv * (dim + vdim);
    float temp = 1.0f;
    if (temp_coef != 0.0f) temp = fmaf(temp_coef, logf((float)((pos + 1) / temp_every + 1)), 1.0f);
    const int n_out = (nq + (writes_cache ? 2 * nkv : 0)) * pad;
    if (by4) {
        // four neighbouring elements of one head a thread (pad, dim and vdim are multiples of four)
        const size_t kv_row = writes_cache ? kv_offset(cache, slot, pos, 0) : 0;
        const size_t kv_head = (size_t)cache.page_size * pad;  // from one kv head's tile to the next
        for (int o = 4 * (blockIdx.y * blockDim.x + threadIdx.x); o < n_out; o += 4 * gridDim.y * blockDim.x) {
            const int head = o / pad, e = o % pad;
            float4 y = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (head < nq) {
                if (e < dim) {
                    y = conv4_at(proj, ld, 0, head * dim + e, bias, w, taps, tail, C, r, before);
                    y.x *= temp; y.y *= temp; y.z *= temp; y.w *= temp;
                }
                store4(q_out + ((size_t)r * nq + head) * pad + e, y);
            } else if (head < nq + nkv) {
                const int kvh = head - nq;
                if (e < dim) y = conv4_at(proj, ld, 0, nq * dim + kvh * dim + e, bias, w, taps, tail, C, r, before);
                store4(k_pages + kv_row + kvh * kv_head + e, y);
            } else {
                const int kvh = head - nq - nkv;
                if (e < vdim)
                    y = conv4_at(proj, ld, 0, (nq + nkv) * dim + kvh * vdim + e, bias, w, taps, tail, C, r, before);
                store4(v_pages + kv_row + kvh * kv_head + e, y);
            }
        }
        return;
    }
    for (int o = blockIdx.y * blockDim.x + threadIdx.x; o < n_out; o += gridDim.y * blockDim.x) {
        const int head = o / pad, e = o % pad;
        if (head < nq) {
            float y = 0.0f;
            if (e < dim) y = conv_at(proj, ld, 0, head * dim + e, bias, w, taps, tail, C, r, before) * temp;
            rfx::st<TO>(q_out, ((size_t)r * nq + head) * pad + e, y);
        } else if (head < nq + nkv) {
            const int kvh = head - nq;
            float y = 0.0f;
            if (e < dim) y = conv_at(proj, ld, 0, nq * dim + kvh * dim + e, bias, w, taps, tail, C, r, before);
            rfx::st<TO>(k_pages, kv_offset(cache, slot, pos, kvh) + e, y);
        } else {
            const int kvh = head - nq - nkv;
            float y = 0.0f;
            if (e < vdim)
                y = conv_at(proj, ld, 0, (nq + nkv) * dim + kvh * vdim + e, bias, w, taps, tail, C, r, before);
            rfx::st<TO>(v_pages, kv_offset(cache, slot, pos, kvh) + e, y);
        }
    }
}

// state[slot][i] <- the input at local time n - T + i (i = 0 .. T - 1): one of
// this step's rows, or what the state held n places later.  A thread owns a
// channel and goes through i upwards, so it reads index n + i > i before
// anything overwrites it.
__global__ void __launch_bounds__(256)
conv_state_update_kernel(const float* __restrict__ proj, int ld, int col0, const float* __restrict__ bias,
                         int taps, float* __restrict__ state, size_t slot_stride,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_row0, int C) {
    pdl_prologue();
    const int s = blockIdx.x;
    const int T = taps - 1;
    const int row0 = seq_row0[s], n = seq_row0[s + 1] - row0;
    float* tail = state + (size_t)seq_slot[s] * slot_stride;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < C; c += gridDim.y * blockDim.x) {
        const float b = bias ? bias[c] : 0.0f;
        for (int i = 0; i < T; ++i) {
            const int src = n - T + i;
            tail[(size_t)i * C + c] = src >= 0 ? proj[(size_t)(row0 + src) * ld + col0 + c] + b
                                             : tail[(size_t)(n + i) * C + c];
        }
    }
}

int chunks(int n, int threads) {
    int g = (n + threads - 1) / threads;
    return g < 1 ? 1 : (g > 64 ? 64 : g);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

// `w`: the filters transposed, [taps][C].  `out_lo` (may be null): the result once
// more, rounded to bfloat16 (the input of a tensor-core product).
// `act`: 0 the convolution as it is, 1 silu of it (after `cbias`).  `update` 1: every
// sequence has exactly one of the R rows, and its last taps - 1 inputs in `state` move on
// by that row in the same launch (what rfx_conv_state_update does for longer steps).
extern "C" int rfx_short_conv_act(const float* proj, int ld, int col0, const float* bias, const float* w,
                                  const float* cbias, int taps, const float* state, long long slot_stride,
                                  const int* row_slot, float* out, void* out_lo, int R, int C, int act,
                                  int update, void* stream) {
    if (R <= 0 || C <= 0) return 0;
    if (act != 0 && act != 1) return RFX_ERR_BAD_ARG;
    if (taps < 1 || taps > MAX_TAPS || (taps > 1 && !state)) return RFX_ERR_BAD_ARG;
    const int by4 = C % 4 == 0 && ld % 4 == 0 && col0 % 4 == 0 && slot_stride % 4 == 0 && aligned16(proj) &&
                    aligned16(bias) && aligned16(w) && aligned16(cbias) && aligned16(state) && aligned16(out) &&
                    ((reinterpret_cast<uintptr_t>(out_lo) & 7) == 0);
    // by fours, many rows: two units a thread share the row's own work; few rows: a unit a thread,
    // so that a decode step's loads are all in flight at once
    dim3 grid(R, chunks(by4 ? C / (R >= 256 ? 8 : 4) : C, 256));
    RFX_LAUNCH(short_conv_kernel, grid, 256, 0, (cudaStream_t)stream, proj, ld, col0, bias, w, cbias, taps,
               const_cast<float*>(state), (size_t)slot_stride, row_slot, out, (__nv_bfloat16*)out_lo, C, by4, act,
               update);
    return 0;
}

extern "C" int rfx_short_conv(const float* proj, int ld, int col0, const float* bias, const float* w,
                              const float* cbias, int taps, const float* state, long long slot_stride,
                              const int* row_slot, float* out, void* out_lo, int R, int C, void* stream) {
    return rfx_short_conv_act(proj, ld, col0, bias, w, cbias, taps, state, slot_stride, row_slot, out, out_lo, R,
                              C, 0, 0, stream);
}

extern "C" int rfx_conv_qkv_post(const float* proj, int ld, const float* bias, const float* w, int taps,
                                 const float* state, long long slot_stride, const int* row_pos,
                                 const int* row_slot, void* q_out, void* k_pages, void* v_pages, int out_dt,
                                 const int* page_table, int max_pages, int page_size, int R, int nq, int nkv,
                                 int dim, int vdim, int pad, float temp_coef, int temp_every,
                                 int writes_cache, void* stream) {
    if (R <= 0) return 0;
    if (taps < 1 || taps > MAX_TAPS || (taps > 1 && !state) || pad < dim || pad < vdim || nkv <= 0 ||
        nq % nkv != 0 || (temp_coef != 0.0f && temp_every <= 0))
        return RFX_ERR_BAD_ARG;
    PagedKV cache{page_table, max_pages, page_size, nkv, pad};
    const int by4 = dim % 4 == 0 && vdim % 4 == 0 && pad % 4 == 0 && ld % 4 == 0 && slot_stride % 4 == 0 &&
                    aligned16(proj) && aligned16(bias) && aligned16(w) && aligned16(state) && aligned16(q_out) &&
                    aligned16(k_pages) && aligned16(v_pages);
    dim3 grid(R, chunks((nq + 2 * nkv) * pad / (by4 ? (R >= 256 ? 8 : 4) : 1), 256));  // as in rfx_short_conv
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dt == RFX_DT_F32)
        RFX_LAUNCH(conv_qkv_post_kernel<float>, grid, 256, 0, s, proj, ld, bias, w, taps, state,
                   (size_t)slot_stride, row_pos, row_slot, (float*)q_out, (float*)k_pages, (float*)v_pages,
                   cache, nq, nkv, dim, vdim, pad, temp_coef, temp_every, writes_cache, by4);
    else if (out_dt == RFX_DT_BF16)
        RFX_LAUNCH(conv_qkv_post_kernel<__nv_bfloat16>, grid, 256, 0, s, proj, ld, bias, w, taps, state,
                   (size_t)slot_stride, row_pos, row_slot, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pages,
                   (__nv_bfloat16*)v_pages, cache, nq, nkv, dim, vdim, pad, temp_coef, temp_every,
                   writes_cache, by4);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_conv_state_update(const float* proj, int ld, int col0, const float* bias, int taps,
                                     float* state, long long slot_stride, const int* seq_slot,
                                     const int* seq_row0, int S, int C, void* stream) {
    if (S <= 0 || C <= 0 || taps <= 1) return 0;
    if (taps > MAX_TAPS) return RFX_ERR_BAD_ARG;
    dim3 grid(S, chunks(C, 256));
    RFX_LAUNCH(conv_state_update_kernel, grid, 256, 0, (cudaStream_t)stream, proj, ld, col0, bias, taps,
               state, (size_t)slot_stride, seq_slot, seq_row0, C);
    return 0;
}
