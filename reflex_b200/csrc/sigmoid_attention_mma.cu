// Attention with sigmoid weights on tensor cores (bfloat16, mma.sync m16n8k16):
// out = sum over the visible keys j of sigmoid((q . K_j) * scale + bias[head]) V_j
// for a packed batch of sequences over the paged cache, prompts, portions and
// decode rows alike.
//
// A CTA serves one (sequence, kv head, tile of query positions).  Its 128 MMA
// rows are (position, head of the kv head's group) pairs, position-major, so the
// pages of that kv head are read once for all heads of the group; each of the 8
// warps owns 16 rows; pages of 64 keys stream through double-buffered
// shared-memory tiles.  Per page a warp makes S = Q K^T, turns every visible
// score into its sigmoid (32-bit; base-2 exponential of the pre-scaled score),
// and adds P V to its accumulators: there is no running maximum, no denominator
// and no rescaling.  Keys are `d` wide and values `dv`; the tiles' columns are
// padded with zeros to DP and DVP, the template's sizes, so that a handful of
// instances serve every head size that is a multiple of 8.
#include "attn_mma.cuh"
#include "common.cuh"

namespace {

using namespace attn;

constexpr int PAGE = 64;
constexpr int SG_THREADS = 256;
constexpr int SG_ROWS = 128;

// rows of `d` elements (d % 8 == 0) into a tile of DP columns (+ 8 of padding): columns
// beyond d and rows beyond rows_valid are zero-filled
template <int DP>
__device__ __forceinline__ void load_tile_pad(__nv_bfloat16* smem, const __nv_bfloat16* gmem, int d, int rows,
                                              int rows_valid, int tid, int nthreads) {
    constexpr int CPR = DP / 8;
    for (int i = tid; i < rows * CPR; i += nthreads) {
        const int r = i / CPR, c = i % CPR;
        const bool ok = r < rows_valid && c * 8 < d;
        cp_async_16(smem + r * (DP + 8) + c * 8, ok ? gmem + (size_t)r * d + c * 8 : gmem, ok);
    }
}

template <int DP, int DVP>
__global__ void __launch_bounds__(SG_THREADS)
attention_sigmoid_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                             const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ page_table,
                             int max_pages, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                             const int* __restrict__ seq_new, const int* __restrict__ seq_row0,
                             __nv_bfloat16* __restrict__ out, int nq, int nkv, int d, int dv, int bq, int window,
                             float scale_log2, const float* __restrict__ bias) {
    constexpr int LD = DP + 8, LDV = DVP + 8, NT = 8;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __nv_bfloat16* qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [128][LD]
    __nv_bfloat16* kbuf = qs + SG_ROWS * LD;                          // [2][PAGE][LD]
    __nv_bfloat16* vbuf = kbuf + 2 * PAGE * LD;                       // [2][PAGE][LDV]

    rfx::pdl_prologue();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = blockIdx.y, kvh = blockIdx.z;
    const int n_new = seq_new[seq];
    const int q0 = (gridDim.x - 1 - blockIdx.x) * bq;  // the latest tiles see the most keys: handed out first
    if (q0 >= n_new) return;
    const int g = nq / nkv;
    const int slot = seq_slot[seq], start = seq_start[seq], row0 = seq_row0[seq];
    const int n_pos = min(bq, n_new - q0);
    const int n_rows = n_pos * g;
    const int pos_first = start + q0, pos_last = pos_first + n_pos - 1;
    const int lo_tile = (window > 0 && pos_first + 1 > window) ? pos_first + 1 - window : 0;

    for (int i = tid; i < SG_ROWS * (DP / 8); i += SG_THREADS) {
        const int row = i / (DP / 8), c = i % (DP / 8);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_rows && c * 8 < d) {
            const int p = row / g, h = row % g;
            v = *reinterpret_cast<const uint4*>(q + ((size_t)(row0 + q0 + p) * nq + kvh * g + h) * d + c * 8);
        }
        *reinterpret_cast<uint4*>(qs + row * LD + c * 8) = v;
    }

    const int* table = page_table + (size_t)slot * max_pages;
    auto issue = [&](int pg, int buf) {
        const size_t tile = ((size_t)table[pg] * nkv + kvh) * PAGE;
        const int valid = min(PAGE, pos_last + 1 - pg * PAGE);
        load_tile_pad<DP>(kbuf + buf * PAGE * LD, k_pages + tile * d, d, PAGE, valid, tid, SG_THREADS);
        load_tile_pad<DVP>(vbuf + buf * PAGE * LDV, v_pages + tile * dv, dv, PAGE, valid, tid, SG_THREADS);
        cp_async_commit();
    };

    // this thread's two rows: warp * 16 + lane / 4 and + 8
    int row_pos[2], row_lo[2];
    float row_bias[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + (lane >> 2) + 8 * h;
        const int p = pos_first + min(row / g, n_pos - 1);
        row_pos[h] = row < n_rows ? p : -1;  // rows beyond the tile see nothing
        row_lo[h] = (window > 0 && p + 1 > window) ? p + 1 - window : 0;
        row_bias[h] = bias ? bias[kvh * g + row % g] * 1.4426950408889634f : 0.0f;
    }
    const int warp_row0 = warp * 16;
    const int warp_pos_max = pos_first + min((min(warp_row0 + 15, n_rows - 1)) / g, n_pos - 1);
    const int warp_pos_min = pos_first + min(warp_row0 / g, n_pos - 1);
    const int warp_lo = (window > 0 && warp_pos_min + 1 > window) ? warp_pos_min + 1 - window : 0;
    const bool warp_active = warp_row0 < n_rows;

    float acc[DVP / 8][4];
#pragma unroll
    for (int n = 0; n < DVP / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;

    const int pg0 = lo_tile / PAGE, pg1 = pos_last / PAGE + 1;
    issue(pg0, 0);
    for (int pg = pg0; pg < pg1; ++pg) {
        const int buf = (pg - pg0) & 1;
        if (pg + 1 < pg1) {
            issue(pg + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int base = pg * PAGE;
        if (warp_active && base <= warp_pos_max && base + PAGE > warp_lo) {
            const __nv_bfloat16* qw = qs + warp_row0 * LD;
            const __nv_bfloat16* ks = kbuf + buf * PAGE * LD;
            const __nv_bfloat16* vs = vbuf + buf * PAGE * LDV;
            float s[NT][4];
#pragma unroll
            for (int t = 0; t < NT; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) s[t][i] = 0.0f;
#pragma unroll
            for (int k0 = 0; k0 < DP; k0 += 16) {
                uint32_t a[4];
                ldmatrix_x4(a, qw + ((lane & 7) + 8 * ((lane >> 3) & 1)) * LD + k0 + 8 * (lane >> 4));
#pragma unroll
                for (int t = 0; t < NT; t += 2) {
                    uint32_t b[4];
                    ldmatrix_x4(b, ks + (t * 8 + (lane & 7) + 8 * (lane >> 4)) * LD + k0 + 8 * ((lane >> 3) & 1));
                    mma_bf16(s[t], a, b[0], b[1]);
                    mma_bf16(s[t + 1], a, b[2], b[3]);
                }
            }
            uint32_t p[NT][2];
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                float e[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int j = base + t * 8 + 2 * (lane & 3) + (i & 1);
                    const int h = i >> 1;
                    const bool vis = j <= row_pos[h] && j >= row_lo[h];
                    // sigmoid(x) = 1 / (1 + 2^(-x log2 e))
                    const float x2 = fmaf(s[t][i], scale_log2, row_bias[h]);
                    e[i] = vis ? __fdividef(1.0f, 1.0f + exp2f(-x2)) : 0.0f;
                }
                p[t][0] = pack_bf16(e[0], e[1]);
                p[t][1] = pack_bf16(e[2], e[3]);
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                const uint32_t a[4] = {p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1]};
#pragma unroll
                for (int n = 0; n < DVP / 8; n += 2) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vs + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * LDV + n * 8 +
                                             8 * (lane >> 4));
                    mma_bf16(acc[n], a, b[0], b[1]);
                    mma_bf16(acc[n + 1], a, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp_row0 + (lane >> 2) + 8 * h;
        if (row >= n_rows) continue;
        const int p = row / g, hd = row % g;
        __nv_bfloat16* o = out + ((size_t)(row0 + q0 + p) * nq + kvh * g + hd) * dv + 2 * (lane & 3);
#pragma unroll
        for (int n = 0; n < DVP / 8; ++n) {
            if (n * 8 + 2 * (lane & 3) < dv)  // dv % 8 == 0: a pair is inside or outside as a whole
                *reinterpret_cast<__nv_bfloat162*>(o + n * 8) =
                    __floats2bfloat162_rn(acc[n][2 * h], acc[n][2 * h + 1]);
        }
    }
}

template <int DP, int DVP>
int launch(const void* q, const void* k_pages, const void* v_pages, const int* page_table, int max_pages,
           const int* seq_slot, const int* seq_start, const int* seq_new, const int* seq_row0, void* out, int S,
           int max_new, int nq, int nkv, int d, int dv, int window, float scale, const float* bias,
           cudaStream_t s) {
    const int g = nq / nkv;
    if (g > SG_ROWS) return RFX_ERR_UNSUPPORTED;
    const int bq = SG_ROWS / g;
    const size_t smem = ((size_t)(SG_ROWS + 2 * PAGE) * (DP + 8) + (size_t)2 * PAGE * (DVP + 8)) * 2;
    auto kernel = attention_sigmoid_mma_kernel<DP, DVP>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_new + bq - 1) / bq, S, nkv);
    if (grid.y > 65535 || grid.z > 65535) return RFX_ERR_UNSUPPORTED;
    RFX_LAUNCH(kernel, grid, SG_THREADS, smem, s, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages,
               (const __nv_bfloat16*)v_pages, page_table, max_pages, seq_slot, seq_start, seq_new, seq_row0,
               (__nv_bfloat16*)out, nq, nkv, d, dv, bq, window, scale * 1.4426950408889634f, bias);
    return 0;
}

}  // namespace

// bfloat16 q [rows, nq, d] and out [rows, nq, dv] packed by sequence; seq_* describe the
// S sequences of the step (slot, positions already cached, rows in this step, first row).
// The cache must already hold this step's keys and values.  d and dv: multiples of 8, d up
// to 256, dv up to 128; group size nq / nkv up to 128; pages of 64.
extern "C" int rfx_attention_sigmoid_mma(const void* q, const void* k_pages, const void* v_pages,
                                         const int* page_table, int max_pages, int page_size,
                                         const int* seq_slot, const int* seq_start, const int* seq_new,
                                         const int* seq_row0, void* out, int S, int max_new, int nq, int nkv,
                                         int d, int dv, int window, float scale, const float* bias,
                                         void* stream) {
    if (S <= 0 || max_new <= 0) return 0;
    if (page_size != PAGE || nkv <= 0 || nq % nkv != 0) return RFX_ERR_BAD_ARG;
    if (d <= 0 || dv <= 0 || d % 8 || dv % 8 || d > 256 || dv > 128) return RFX_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int dp = d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : 256;
    const int dvp = dv <= 32 ? 32 : dv <= 64 ? 64 : 128;
#define RFX_CASE(A, B)                                                                                      \
    if (dp == A && dvp == B)                                                                                \
        return launch<A, B>(q, k_pages, v_pages, page_table, max_pages, seq_slot, seq_start, seq_new,       \
                            seq_row0, out, S, max_new, nq, nkv, d, dv, window, scale, bias, s);
    RFX_CASE(32, 32) RFX_CASE(32, 64) RFX_CASE(32, 128) RFX_CASE(64, 32) RFX_CASE(64, 64) RFX_CASE(64, 128)
    RFX_CASE(128, 32) RFX_CASE(128, 64) RFX_CASE(128, 128) RFX_CASE(256, 32) RFX_CASE(256, 64) RFX_CASE(256, 128)
#undef RFX_CASE
    return RFX_ERR_UNSUPPORTED;
}
