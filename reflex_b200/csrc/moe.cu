// Mixture-of-experts feed-forward with top-k routing, for any number of rows.
//
//  * rfx_moe_route: router logits (32-bit, bias added here) -> the `top`
//    experts with the largest logits (ties: the lower index) and their weights:
//    the softmax over the chosen logits only (mode 0), or each chosen logit's
//    sigmoid, not renormalised (mode 1), or the softmax over all experts with the
//    chosen ones' scores renormalised by their sum (mode 2); rfx_moe_route_scaled
//    also multiplies the weights by a constant.  One warp a row.
//  * rfx_moe_up: act[(r, k), :] = f(W_up[e] (s x[r])) for expert e = ids[r, k];
//    f = relu squared (act 0) or silu (act 1); act 2 is the gated, clamped form
//    over W_up[e] = [gate rows | up rows]: g' = min(g, limit), u' = clamp(u,
//    -limit, limit), g' sigmoid(alpha g') (u' + 1); act 3 the gated silu over the
//    same layout, silu(g) u.  `in_scale` (may be null)
//    gives s per (row, choice): a weight on the expert's input.  One warp an
//    output element, the row in shared memory.
//  * rfx_moe_down: y[r, :] = sum_k wts[r, k] W_down[ids[r, k]] act[(r, k), :],
//    the experts in the order of their rank, 32-bit sums: a row's result does
//    not depend on the batch.  Null `wts`: every weight is one.
//  * Many rows (prefill): rfx_moe_group places the (row, choice) pairs expert by
//    expert (counts, offsets, each pair's place), rfx_moe_gather copies the
//    rows into that order, the library multiplies each expert's block by its
//    matrices, rfx_moe_activation applies f in place, and rfx_moe_combine sums
//    a row's `top` results in the order of their rank with their weights.
// Expert weights are stacked: W_up [experts, ff, width], W_down [experts, width, ff].
#include "common.cuh"

namespace {

using namespace rfx;

constexpr int MAX_PER_LANE = 8;  // up to 256 experts

__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                 int* __restrict__ ids, float* __restrict__ wts, int R, int E, int top,
                                 int mode, float scale) {
    pdl_prologue();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= R) return;
    float z[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int e = i * 32 + lane;
        z[i] = e < E ? logits[(size_t)r * ld + e] + (bias ? bias[e] : 0.0f) : -INFINITY;
    }
    float zmax = 0.0f, sum = mode == 1 ? 1.0f : 0.0f, mine = 0.0f;  // lane k keeps the k-th choice's exponential
    int my_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int e = i * 32 + lane;
            if (z[i] > best) { best = z[i]; best_e = e; }  // within a lane e rises: the lower index wins a tie
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        if (k == 0) zmax = best;
        // mode 1: the chosen logit's sigmoid is the weight as it is (sum stays one)
        const float p = mode == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - zmax);
        if (mode != 1) sum += p;
        if ((k & 31) == lane && k < 32) { mine = p; my_id = best_e; }
        if (k >= 32 && lane == 0) {  // more than 32 choices: written unnormalised, scaled below
            ids[(size_t)r * top + k] = best_e;
            wts[(size_t)r * top + k] = p;
        }
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i)
            if (i * 32 + lane == best_e) z[i] = -INFINITY;
    }
    if (mode == 2) {
        // scores are the softmax over all experts; the chosen ones' scores over their sum
        // (+ 1e-20), times `scale`.  z holds -inf where an expert was chosen: the others'
        // exponentials join the chosen ones' for the softmax's denominator
        float rest = 0.0f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i)
            if (i * 32 + lane < E && z[i] != -INFINITY) rest += expf(z[i] - zmax);
        const float total = sum + warp_sum(rest);
        const float chosen = sum / total + 1e-20f;
        if (lane < top) {
            ids[(size_t)r * top + lane] = my_id;
            wts[(size_t)r * top + lane] = (mine / total) / chosen * scale;
        }
        if (lane == 0)
            for (int k = 32; k < top; ++k) wts[(size_t)r * top + k] = (wts[(size_t)r * top + k] / total) / chosen * scale;
        return;
    }
    if (lane < top) {
        ids[(size_t)r * top + lane] = my_id;
        wts[(size_t)r * top + lane] = mine / sum * scale;
    }
    if (lane == 0)
        for (int k = 32; k < top; ++k) wts[(size_t)r * top + k] = wts[(size_t)r * top + k] / sum * scale;
}

// sum_c xs[c] * w[c] over a warp; bfloat16 rows that start on 16 bytes go eight
// elements a load.  The order depends on n and the row's alignment alone.
template <typename T>
__device__ __forceinline__ float warp_dot(const float* __restrict__ xs, const T* __restrict__ w, int n,
                                          int lane) {
    float dot = 0.0f;
    int c0 = 0;
    if constexpr (sizeof(T) == 2) {
        if ((n & 7) == 0 && ((reinterpret_cast<uintptr_t>(w) | (uintptr_t)__cvta_generic_to_shared(xs)) & 15) == 0) {
            const uint4* w8 = reinterpret_cast<const uint4*>(w);
            const int n8 = n / 8;
            for (int v0 = lane; v0 < n8; v0 += 128) {  // four loads in flight a lane
                uint4 u[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    u[j] = v0 + 32 * j < n8 ? w8[v0 + 32 * j] : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (v0 + 32 * j >= n8) break;
                    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u[j]);
                    const float4* xv = reinterpret_cast<const float4*>(xs + 8 * (v0 + 32 * j));
                    const float4 x0 = xv[0], x1 = xv[1];
                    const float2 f0 = __bfloat1622float2(p[0]), f1 = __bfloat1622float2(p[1]);
                    const float2 f2 = __bfloat1622float2(p[2]), f3 = __bfloat1622float2(p[3]);
                    dot = fmaf(x0.x, f0.x, dot);
                    dot = fmaf(x0.y, f0.y, dot);
                    dot = fmaf(x0.z, f1.x, dot);
                    dot = fmaf(x0.w, f1.y, dot);
                    dot = fmaf(x1.x, f2.x, dot);
                    dot = fmaf(x1.y, f2.y, dot);
                    dot = fmaf(x1.z, f3.x, dot);
                    dot = fmaf(x1.w, f3.y, dot);
                }
            }
            c0 = n / 8 * 8;
        }
    }
    for (int c = c0 + lane; c < n; c += 32) dot = fmaf(xs[c], ld<T>(w, c), dot);
    return warp_sum(dot);
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_up_kernel(const T* __restrict__ x, const T* __restrict__ W, const int* __restrict__ ids,
              const float* __restrict__ in_scale, T* __restrict__ act, int top, int ff, int width, int kind,
              float alpha, float limit) {
    extern __shared__ __align__(16) float xs[];  // the row
    pdl_prologue();
    const int pair = blockIdx.x;
    const int r = pair / top;
    const int e = ids[pair];
    // a weight on the expert's input; the scaled row is rounded to the storage type,
    // as the rows of the grouped form are
    const float sc = in_scale ? in_scale[pair] : 1.0f;
    for (int c = threadIdx.x; c < width; c += blockDim.x) {
        const float v = ld<T>(x, (size_t)r * width + c);
        if (in_scale) {
            if constexpr (sizeof(T) == 2) xs[c] = __bfloat162float(__float2bfloat16_rn(v * sc));
            else xs[c] = v * sc;
        } else xs[c] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const T* We = W + (size_t)e * (kind >= 2 ? 2 : 1) * ff * width;
    for (int j = blockIdx.y * nwarps + warp; j < ff; j += gridDim.y * nwarps) {
        const T* wrow = We + (size_t)j * width;
        const float dot = warp_dot<T>(xs, wrow, width, lane);
        if (kind == 3) {  // gated silu over [gate rows | up rows]
            const float up = warp_dot<T>(xs, wrow + (size_t)ff * width, width, lane);
            if (lane == 0) st<T>(act, (size_t)pair * ff + j, (dot / (1.0f + expf(-dot))) * up);
        } else if (kind == 2) {
            const float up = warp_dot<T>(xs, wrow + (size_t)ff * width, width, lane);
            if (lane == 0) {
                const float g = fminf(dot, limit), u = fminf(fmaxf(up, -limit), limit);
                st<T>(act, (size_t)pair * ff + j, (g / (1.0f + expf(-alpha * g))) * (u + 1.0f));
            }
        } else if (lane == 0) {
            float a;
            if (kind == 0) { a = fmaxf(dot, 0.0f); a *= a; }
            else a = dot / (1.0f + expf(-dot));
            st<T>(act, (size_t)pair * ff + j, a);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_down_kernel(const T* __restrict__ act, const T* __restrict__ W, const int* __restrict__ ids,
                const float* __restrict__ wts, float* __restrict__ y, int top, int ff, int width) {
    extern __shared__ __align__(16) float as[];  // [top][ff]
    pdl_prologue();
    const int r = blockIdx.x;
    for (int c = threadIdx.x; c < top * ff; c += blockDim.x) as[c] = ld<T>(act, (size_t)r * top * ff + c);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int n = blockIdx.y * nwarps + warp; n < width; n += gridDim.y * nwarps) {
        float total = 0.0f;
        for (int k = 0; k < top; ++k) {
            const T* wrow = W + ((size_t)ids[(size_t)r * top + k] * width + n) * ff;
            total = fmaf(wts ? wts[(size_t)r * top + k] : 1.0f, warp_dot<T>(as + k * ff, wrow, ff, lane), total);
        }
        if (lane == 0) y[(size_t)r * width + n] = total;
    }
}

// One block: counts per expert, offsets (exclusive prefix, [E + 1]) and each
// pair's place in the expert-by-expert order.  Places within an expert are
// handed out as the threads arrive; a pair's result does not depend on its place.
__global__ void __launch_bounds__(1024)
moe_group_kernel(const int* __restrict__ ids, int n_pairs, int E, int* __restrict__ offsets,
                 int* __restrict__ place) {
    extern __shared__ int cnt[];  // [E] counts, then [E] cursors
    int* cursor = cnt + E;
    pdl_prologue();
    for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[ids[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += cnt[e];
        }
        offsets[E] = run;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) place[p] = atomicAdd(&cursor[ids[p]], 1);
}

// xg[place[p], :] = x[p / top, :] (times scale[p], when given)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ place,
                                  const float* __restrict__ scale, T* __restrict__ xg, int top, int width) {
    pdl_prologue();
    const int p = blockIdx.x;
    const T* src = x + (size_t)(p / top) * width;
    T* dst = xg + (size_t)place[p] * width;
    const int bytes = width * (int)sizeof(T);
    if (scale) {
        const float sc = scale[p];
        if constexpr (sizeof(T) == 2) {
            if ((bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
                // eight elements a thread and step
                for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width / 8; c += gridDim.y * blockDim.x) {
                    uint4 v = reinterpret_cast<const uint4*>(src)[c];
                    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        h[j] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
                    }
                    reinterpret_cast<uint4*>(dst)[c] = v;
                }
                return;
            }
        }
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x)
            st<T>(dst, c, ld<T>(src, c) * sc);
    } else if (blockIdx.y > 0) {
        return;  // the plain copy is one block's
    } else if ((bytes & 15) == 0 && ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
        for (int c = threadIdx.x; c < bytes / 16; c += blockDim.x)
            reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
    }
}

template <typename T>
__global__ void moe_activation_kernel(T* __restrict__ a, size_t n, int kind) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float z = ld<T>(a, i);
        float v;
        if (kind == 0) { v = fmaxf(z, 0.0f); v *= v; }
        else v = z / (1.0f + expf(-z));
        st<T>(a, i, v);
    }
}

// the same for bfloat16, eight elements (16 bytes) a thread and step; n8 = n / 8
__global__ void moe_activation_bf16x8_kernel(uint4* __restrict__ a, size_t n8, int kind) {
    pdl_prologue();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        uint4 v = a[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 z = __bfloat1622float2(h[j]);
            if (kind == 0) {
                z.x = fmaxf(z.x, 0.0f); z.x *= z.x;
                z.y = fmaxf(z.y, 0.0f); z.y *= z.y;
            } else {
                z.x = z.x / (1.0f + expf(-z.x));
                z.y = z.y / (1.0f + expf(-z.y));
            }
            h[j] = __floats2bfloat162_rn(z.x, z.y);
        }
        a[i] = v;
    }
}

// y[r, :] = sum_k wts[r, k] * yg[place[r * top + k], :], k in order
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ yg, const int* __restrict__ place,
                                   const float* __restrict__ wts, float* __restrict__ y, int top, int width) {
    pdl_prologue();
    const int r = blockIdx.x;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < width; c += gridDim.y * blockDim.x) {
        float total = 0.0f;
        for (int k = 0; k < top; ++k)
            total = fmaf(wts ? wts[(size_t)r * top + k] : 1.0f,
                         ld<T>(yg, (size_t)place[(size_t)r * top + k] * width + c), total);
        y[(size_t)r * width + c] = total;
    }
}

}  // namespace

extern "C" int rfx_moe_group(const int* ids, int n_pairs, int E, int* offsets, int* place, void* stream) {
    if (n_pairs <= 0 || E <= 0) return RFX_ERR_BAD_ARG;
    if (E > 8192) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(moe_group_kernel, 1, 1024, (size_t)2 * E * sizeof(int), (cudaStream_t)stream, ids, n_pairs, E,
               offsets, place);
    return 0;
}

extern "C" int rfx_moe_gather(const void* x, const int* place, const float* scale, void* xg, int dt,
                              int n_pairs, int top, int width, void* stream) {
    if (n_pairs <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    // a scaled copy of few rows: a thread an element, so that every load is in flight at once
    int gy = 1;
    if (scale) {
        gy = (width + 127) / 128;
        const int most = sm_count() * 8 / n_pairs;
        if (gy > most) gy = most;
        if (gy < 1) gy = 1;
    }
    dim3 grid(n_pairs, gy);
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(moe_gather_kernel<float>, grid, 128, 0, s, (const float*)x, place, scale, (float*)xg, top,
                   width);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(moe_gather_kernel<__nv_bfloat16>, grid, 128, 0, s, (const __nv_bfloat16*)x, place, scale,
                   (__nv_bfloat16*)xg, top, width);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_moe_activation(void* a, int dt, long long n, int kind, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int blocks = (int)((n + 255) / 256);
    if (blocks > sm_count() * 16) blocks = sm_count() * 16;
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(moe_activation_kernel<float>, blocks, 256, 0, s, (float*)a, (size_t)n, kind);
    else if (dt == RFX_DT_BF16 && n % 8 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0) {
        int blocks8 = (int)((n / 8 + 255) / 256);
        if (blocks8 > sm_count() * 16) blocks8 = sm_count() * 16;
        RFX_LAUNCH(moe_activation_bf16x8_kernel, blocks8, 256, 0, s, (uint4*)a, (size_t)(n / 8), kind);
    } else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(moe_activation_kernel<__nv_bfloat16>, blocks, 256, 0, s, (__nv_bfloat16*)a, (size_t)n, kind);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

extern "C" int rfx_moe_combine(const void* yg, int dt, const int* place, const float* wts, float* y, int R,
                               int top, int width, void* stream) {
    if (R <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    int gy = (width + 255) / 256;  // few rows: a thread an element
    const int most = sm_count() * 8 / R;
    if (gy > most) gy = most;
    if (gy < 1) gy = 1;
    dim3 grid(R, gy);
    if (dt == RFX_DT_F32)
        RFX_LAUNCH(moe_combine_kernel<float>, grid, 256, 0, s, (const float*)yg, place, wts, y, top, width);
    else if (dt == RFX_DT_BF16)
        RFX_LAUNCH(moe_combine_kernel<__nv_bfloat16>, grid, 256, 0, s, (const __nv_bfloat16*)yg, place, wts, y, top,
                   width);
    else
        return RFX_ERR_BAD_ARG;
    return 0;
}

// `ld`: floats between two rows of `logits` (>= E: further columns are ignored)
// mode 2: the softmax over all experts, the chosen ones' scores over their sum (+ 1e-20);
// `scale` multiplies the weights of every mode
extern "C" int rfx_moe_route_scaled(const float* logits, int ld, const float* bias, int* ids, float* wts, int R,
                                    int E, int top, int mode, float scale, void* stream) {
    if (R <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || ld < E || mode < 0 || mode > 2) return RFX_ERR_BAD_ARG;
    if (E > 32 * MAX_PER_LANE) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(moe_route_kernel, (R + 3) / 4, 128, 0, (cudaStream_t)stream, logits, ld, bias, ids, wts, R, E, top,
               mode, scale);
    return 0;
}

extern "C" int rfx_moe_route(const float* logits, int ld, const float* bias, int* ids, float* wts, int R, int E,
                             int top, int mode, void* stream) {
    if (mode != 0 && mode != 1) return RFX_ERR_BAD_ARG;
    return rfx_moe_route_scaled(logits, ld, bias, ids, wts, R, E, top, mode, 1.0f, stream);
}

extern "C" int rfx_moe_up(const void* x, const void* W, const int* ids, const float* in_scale, void* act, int dt,
                          int R, int top, int ff, int width, int kind, float alpha, float limit, void* stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    int gy = (ff + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(R * top, gy);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(T)                                                                                        \
    do {                                                                                                 \
        if (smem > 48 * 1024) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(moe_up_kernel<T>,                                       \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                         \
        }                                                                                                \
        RFX_LAUNCH(moe_up_kernel<T>, grid, 256, smem, s, (const T*)x, (const T*)W, ids, in_scale, (T*)act, \
                   top, ff, width, kind, alpha, limit);                                                  \
    } while (0)
    if (dt == RFX_DT_F32) RFX_GO(float);
    else if (dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}

extern "C" int rfx_moe_down(const void* act, const void* W, const int* ids, const float* wts, float* y,
                            int dt, int R, int top, int ff, int width, void* stream) {
    if (R <= 0) return 0;
    const size_t smem = (size_t)top * ff * sizeof(float);
    if (smem > 200 * 1024) return RFX_ERR_UNSUPPORTED;
    int gy = (width + 7) / 8;
    if (gy > 64) gy = 64;
    dim3 grid(R, gy);
    cudaStream_t s = (cudaStream_t)stream;
#define RFX_GO(T)                                                                                        \
    do {                                                                                                 \
        if (smem > 48 * 1024) {                                                                          \
            cudaError_t e = cudaFuncSetAttribute(moe_down_kernel<T>,                                     \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e;                                                         \
        }                                                                                                \
        RFX_LAUNCH(moe_down_kernel<T>, grid, 256, smem, s, (const T*)act, (const T*)W, ids, wts, y, top,   \
                   ff, width);                                                                           \
    } while (0)
    if (dt == RFX_DT_F32) RFX_GO(float);
    else if (dt == RFX_DT_BF16) RFX_GO(__nv_bfloat16);
    else return RFX_ERR_BAD_ARG;
#undef RFX_GO
    return 0;
}
