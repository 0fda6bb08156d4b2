// Hyper-connections: the residual as S parallel copies ("streams") of the
// model's width, 32-bit, [rows][S][W].
//
// A sublayer reads u = sum_s in[s] x_s and, with its result y (times a
// per-channel scale ls), every copy is rewritten at once from the old ones:
//     x_t <- sum_s mix[s][t] x_s + out[t] * (ls * y)        (mix is [from][to])
// S = 1 with in = out = mix = 1 is the ordinary residual sum x <- x + ls * y.
//
//  * rfx_hyper_expand: the embedding output into all S copies.
//  * rfx_hyper_step: the write of the sublayer before (if there is one), then the
//    read for the next sublayer and its RMS norm,
//        u / sqrt(mean(u^2) + eps) * (offset + w),
//    in one pass over the row: the copies are read once and written once, and
//    the norm needs no launch of its own.  A block owns a row; u stays in shared
//    memory between the sum of squares and the output.
//  * rfx_hyper_collapse: the last write and the sum of the copies, [rows][W].
//
// All arithmetic is 32-bit.  The sums over s run in index order.
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int MAX_S = 8;

struct Coef {
    float in[MAX_S];
    float out[MAX_S];
    float mix[MAX_S * MAX_S];
};

// the S new values of column c of a row: reads the old copies, applies the write
template <typename TY>
__device__ __forceinline__ void rewrite(const float* __restrict__ xrow, int S, int W, int c, const TY* __restrict__ yrow,
                                        const float* __restrict__ ls, const float* mix, const float* outw,
                                        float (&x)[MAX_S]) {
    float old[MAX_S];
#pragma unroll
    for (int s = 0; s < MAX_S; ++s) old[s] = s < S ? xrow[(size_t)s * W + c] : 0.0f;
    if (yrow == nullptr) {
#pragma unroll
        for (int s = 0; s < MAX_S; ++s) x[s] = old[s];
        return;
    }
    const float y = ls ? ld<TY>(yrow, c) * ls[c] : ld<TY>(yrow, c);
#pragma unroll
    for (int t = 0; t < MAX_S; ++t) {
        float v = 0.0f;
        if (t < S) {
            for (int s = 0; s < S; ++s) v = fmaf(mix[s * S + t], old[s], v);
            v = fmaf(outw[t], y, v);
        }
        x[t] = v;
    }
}

__global__ void __launch_bounds__(256)
hyper_expand_kernel(const float* __restrict__ x, float* __restrict__ streams, int S, int W) {
    pdl_prologue();
    const size_t r = blockIdx.x;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = x[r * W + c];
        for (int s = 0; s < S; ++s) streams[(r * S + s) * W + c] = v;
    }
}

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
hyper_step_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ ls,
                  const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ in,
                  const float* __restrict__ norm_w, float eps, float w_offset, TO* __restrict__ out, int S, int W) {
    extern __shared__ float u_row[];  // [W]
    __shared__ float scratch[32];
    __shared__ Coef cf;
    pdl_launch_dependents();
    // the coefficients are weights: no kernel writes them
    if (threadIdx.x < S) {
        cf.in[threadIdx.x] = in[threadIdx.x];
        if (y) cf.out[threadIdx.x] = outw[threadIdx.x];
    }
    if (y && threadIdx.x < S * S) cf.mix[threadIdx.x] = mix[threadIdx.x];
    __syncthreads();
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xrow = streams + r * S * W;
    const TY* yrow = y ? y + r * W : nullptr;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        float x[MAX_S];
        rewrite<TY>(xrow, S, W, c, yrow, ls, cf.mix, cf.out, x);
        float u = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_S; ++s) {
            if (s < S) {
                if (yrow) xrow[(size_t)s * W + c] = x[s];
                u = fmaf(cf.in[s], x[s], u);
            }
        }
        u_row[c] = u;
        ss = fmaf(u, u, ss);
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x)
        st<TO>(out, r * W + c, (u_row[c] * rinv) * (w_offset + norm_w[c]));
}

// The same step, four neighbouring columns a thread and the stream count a
// compile-time number: the copies move as 16-byte accesses and the small sums
// over s unroll.  Per column the arithmetic and its order are those above.
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ float4 fma4(float a, float4 b, float4 c) {
    return make_float4(fmaf(a, b.x, c.x), fmaf(a, b.y, c.y), fmaf(a, b.z, c.z), fmaf(a, b.w, c.w));
}

template <typename TY, typename TO, int S>
__global__ void __launch_bounds__(256)
hyper_step4_kernel(float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ ls,
                   const float* __restrict__ mix, const float* __restrict__ outw, const float* __restrict__ in,
                   const float* __restrict__ norm_w, float eps, float w_offset, TO* __restrict__ out, int W) {
    extern __shared__ float4 u_row4[];  // [W / 4]
    __shared__ float scratch[32];
    __shared__ Coef cf;
    pdl_launch_dependents();
    if (threadIdx.x < S) {
        cf.in[threadIdx.x] = in[threadIdx.x];
        if (y) cf.out[threadIdx.x] = outw[threadIdx.x];
    }
    if (y && threadIdx.x < S * S) cf.mix[threadIdx.x] = mix[threadIdx.x];
    __syncthreads();
    pdl_wait();
    const size_t r = blockIdx.x;
    float* xrow = streams + r * S * W;
    const int W4 = W >> 2;
    float ss = 0.0f;
    for (int c4 = threadIdx.x; c4 < W4; c4 += blockDim.x) {
        const int c = c4 << 2;
        float4 x[S];
#pragma unroll
        for (int s = 0; s < S; ++s) x[s] = load4(xrow + (size_t)s * W + c);
        if (y) {
            float4 yv = load4(y + r * W + c);
            if (ls) {
                const float4 l = load4(ls + c);
                yv = make_float4(yv.x * l.x, yv.y * l.y, yv.z * l.z, yv.w * l.w);
            }
            float4 nx[S];
#pragma unroll
            for (int t = 0; t < S; ++t) {
                float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int s = 0; s < S; ++s) v = fma4(cf.mix[s * S + t], x[s], v);
                nx[t] = fma4(cf.out[t], yv, v);
            }
#pragma unroll
            for (int s = 0; s < S; ++s) {
                x[s] = nx[s];
                store4(xrow + (size_t)s * W + c, x[s]);
            }
        }
        float4 u = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int s = 0; s < S; ++s) u = fma4(cf.in[s], x[s], u);
        u_row4[c4] = u;
        ss = fmaf(u.x, u.x, ss);
        ss = fmaf(u.y, u.y, ss);
        ss = fmaf(u.z, u.z, ss);
        ss = fmaf(u.w, u.w, ss);
    }
    const float total = block_sum(ss, scratch);
    const float rinv = 1.0f / sqrtf(total / (float)W + eps);
    for (int c4 = threadIdx.x; c4 < W4; c4 += blockDim.x) {
        const float4 u = u_row4[c4], w = load4(norm_w + (c4 << 2));
        store4(out + r * W + (c4 << 2),
               make_float4((u.x * rinv) * (w_offset + w.x), (u.y * rinv) * (w_offset + w.y),
                           (u.z * rinv) * (w_offset + w.z), (u.w * rinv) * (w_offset + w.w)));
    }
}

template <typename TY>
__global__ void __launch_bounds__(256)
hyper_collapse_kernel(const float* __restrict__ streams, const TY* __restrict__ y, const float* __restrict__ ls,
                      const float* __restrict__ mix, const float* __restrict__ outw, float* __restrict__ out,
                      const int* __restrict__ rows, int S, int W) {
    __shared__ Coef cf;
    pdl_launch_dependents();
    if (y && threadIdx.x < S) cf.out[threadIdx.x] = outw[threadIdx.x];
    if (y && threadIdx.x < S * S) cf.mix[threadIdx.x] = mix[threadIdx.x];
    __syncthreads();
    pdl_wait();
    const size_t r = rows ? (size_t)rows[blockIdx.x] : blockIdx.x;  // out row blockIdx.x is row r of the streams
    const float* xrow = streams + r * S * W;
    const TY* yrow = y ? y + r * W : nullptr;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < W; c += gridDim.y * blockDim.x) {
        float x[MAX_S];
        rewrite<TY>(xrow, S, W, c, yrow, ls, cf.mix, cf.out, x);
        float sum = 0.0f;
#pragma unroll
        for (int s = 0; s < MAX_S; ++s)
            if (s < S) sum += x[s];
        out[(size_t)blockIdx.x * W + c] = sum;
    }
}

}  // namespace

extern "C" int rfx_hyper_expand(const float* x, float* streams, int R, int S, int W, void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(hyper_expand_kernel, dim3(R), 256, 0, (cudaStream_t)stream, x, streams, S, W);
    return 0;
}

// `y` may be null (no write before the read); `ls` may be null (no per-channel scale).
extern "C" int rfx_hyper_step(float* streams, const void* y, int y_dt, const float* ls, const float* mix,
                              const float* outw, const float* in, const float* norm_w, float eps, float w_offset,
                              void* out, int out_dt, int R, int S, int W, void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0 || (size_t)W * sizeof(float) > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    if (y && (!mix || !outw)) return RFX_ERR_BAD_ARG;
    const size_t smem = (size_t)W * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_HYPER(TY, TO)                                                                                          \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(hyper_step_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        RFX_LAUNCH((hyper_step_kernel<TY, TO>), dim3(R), 256, smem, s, streams, (const TY*)y, ls, mix, outw, in,   \
                   norm_w, eps, w_offset, (TO*)out, S, W);                                                         \
    } while (0)
    const bool y16 = y && y_dt == RFX_DT_BF16;
    auto aligned = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
    if (W % 4 == 0 && (S == 1 || S == 2 || S == 3 || S == 4 || S == 8) && aligned(streams) && aligned(y) &&
        aligned(ls) && aligned(norm_w) && aligned(out)) {
#define RFX_HYPER4(TY, TO, NS)                                                                                  \
    do {                                                                                                        \
        if (smem > 48 * 1024)                                                                                   \
            cudaFuncSetAttribute(hyper_step4_kernel<TY, TO, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                 (int)smem);                                                                    \
        RFX_LAUNCH((hyper_step4_kernel<TY, TO, NS>), dim3(R), 256, smem, s, streams, (const TY*)y, ls, mix,     \
                   outw, in, norm_w, eps, w_offset, (TO*)out, W);                                               \
    } while (0)
#define RFX_HYPER4_S(TY, TO)                    \
    do {                                        \
        if (S == 1) RFX_HYPER4(TY, TO, 1);      \
        else if (S == 2) RFX_HYPER4(TY, TO, 2); \
        else if (S == 3) RFX_HYPER4(TY, TO, 3); \
        else if (S == 4) RFX_HYPER4(TY, TO, 4); \
        else RFX_HYPER4(TY, TO, 8);             \
    } while (0)
        if (out_dt == RFX_DT_F32) {
            if (y16) RFX_HYPER4_S(__nv_bfloat16, float);
            else RFX_HYPER4_S(float, float);
        } else if (out_dt == RFX_DT_BF16) {
            if (y16) RFX_HYPER4_S(__nv_bfloat16, __nv_bfloat16);
            else RFX_HYPER4_S(float, __nv_bfloat16);
        } else {
            return RFX_ERR_BAD_ARG;
        }
#undef RFX_HYPER4_S
#undef RFX_HYPER4
        return 0;
    }
    if (out_dt == RFX_DT_F32) {
        if (y16) RFX_HYPER(__nv_bfloat16, float);
        else RFX_HYPER(float, float);
    } else if (out_dt == RFX_DT_BF16) {
        if (y16) RFX_HYPER(__nv_bfloat16, __nv_bfloat16);
        else RFX_HYPER(float, __nv_bfloat16);
    } else {
        return RFX_ERR_BAD_ARG;
    }
#undef RFX_HYPER
    return 0;
}

// `rows` (may be null): R row indices on the device; out row i is then the sum for row rows[i]
// of the streams (and of `y`), so that only the rows somebody wants are made.
extern "C" int rfx_hyper_collapse(const float* streams, const void* y, int y_dt, const float* ls, const float* mix,
                                  const float* outw, float* out, const int* rows, int R, int S, int W,
                                  void* stream) {
    if (R <= 0) return 0;
    if (S < 1 || S > MAX_S || W <= 0) return RFX_ERR_UNSUPPORTED;
    if (y && (!mix || !outw)) return RFX_ERR_BAD_ARG;
    int gy = (W + 255) / 256;
    if (R >= 64) gy = 1;
    else if (gy > 32) gy = 32;
    cudaStream_t s = (cudaStream_t)stream;
    if (y && y_dt == RFX_DT_BF16)
        RFX_LAUNCH(hyper_collapse_kernel<__nv_bfloat16>, dim3(R, gy), 256, 0, s, streams, (const __nv_bfloat16*)y, ls,
                   mix, outw, out, rows, S, W);
    else
        RFX_LAUNCH(hyper_collapse_kernel<float>, dim3(R, gy), 256, 0, s, streams, (const float*)y, ls, mix, outw,
                   out, rows, S, W);
    return 0;
}
