// Hybrid language-model engine (sm_100a): ragged-batch step over a paged key/value pool and per-sequence recurrent
// state slots.  See include/smoltts_b200_lm.h for what every entry point takes and returns.
//
// Precision: the residual stream, all norms, attention scores / softmax weights and the whole recurrence run in fp32.
// T (bf16 or float) is the element type of matrices, of the inputs of the matrix products and of the key/value pool;
// every matrix product accumulates in fp32 and writes fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/smoltts_b200_lm.h"
#include "common.cuh"
#include "sampler.cuh"
#include "tmap_host.h"
#include "umma.cuh"

#define SMOL_OK 0
#define SMOL_ERR_INVALID (-1)
#define SMOL_ERR_UNBOUND (-2)
#define SMOL_ERR_CUDA (-3)
#define SMOL_ERR_UNSUPPORTED (-4)
#define SMOL_ERR_CAPACITY (-5)

namespace smol {
namespace lm {

template <class T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<bf16>(bf16 v) { return __bfloat162float(v); }
template <class T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

// Sum over the block; every thread gets the result.  `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (l == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = l < nw ? red[l] : 0.0f;
        t = warp_sum(t);
        if (l == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// ---------------------------------------------------------------------------------------------------------------------
// Embedding: x[t] = embed[token[t]] * scale, then the first layer's norm -> hn.  The norms of the sandwich block multiply
// by woff + w: woff = 1 for one-plus weight vectors, 0 for plain ones.
template <class T>
__global__ void embed_norm_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, float scale, int D, int vocab,
                                  const float* __restrict__ wn, float eps, float* __restrict__ x, T* __restrict__ hn, const float woff) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const T* e = embed + (size_t)tok * D;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = to_f<T>(e[c]) * scale;
        x[(size_t)t * D + c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) hn[(size_t)t * D + c] = from_f<T>(x[(size_t)t * D + c] * r * (woff + wn[c]));
}

// RMS norm of selected rows -> T.  rows == nullptr: row r of the output is row r of the input.
template <class T>
__global__ void norm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const float* __restrict__ w, float eps,
                                 int D, T* __restrict__ out, const float woff) {
    __shared__ float red[33];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * D;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) ss += xr[c] * xr[c];
    ss = block_sum(ss, red);
    const float s = 1.0f / sqrtf(ss / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) out[(size_t)r * D + c] = from_f<T>(xr[c] * s * (woff + w[c]));
}

// End of a sublayer fused with the start of the next one:
//   x <- x + ls * (y / rms(y) * (woff + wb));   hn <- x / rms(x) * (woff + wn)     (wn == nullptr: no next norm)
// yb != nullptr: a bias [D] joins y first (the output projection's).  rs.yp != nullptr: y is instead the routed experts'
// weighted sum, taken here (hin: the sublayer's input, which identity outputs hand on).  One block per row; the new row
// is kept in shared memory between the two passes.
constexpr int kRowRegs = 8;   // add_norm keeps a row in registers when it has at most 8 elements per thread

// The sublayer's output of a routed feed-forward, summed on the fly by the norm kernel that follows it: for the `top`
// choices k of a token (ascending), weight[k] * (row slot_of[k] of the experts' outputs, or the token's input itself where
// slot_of[k] < 0: an identity output).  sel_w == nullptr: every weight is 1 (the weights went into the experts' inputs).
struct RoutedSum {
    const float* yp;              // nullptr: the sublayer's output is y
    const int32_t* slot_of;
    const float* sel_w;
    int top;
};

template <class T>
__global__ void add_norm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ wb,
                                const float* __restrict__ ls, const float* __restrict__ wn, float eps, int D, T* __restrict__ hn,
                                const float woff, const float* __restrict__ yb, const RoutedSum rs, const T* hin) {
    extern __shared__ float row[];
    __shared__ float red[33];
    const size_t o = (size_t)blockIdx.x * D;
    auto y_at = [&](int c) -> float {
        if (!rs.yp) return y[o + c] + (yb ? yb[c] : 0.0f);
        float acc = 0.0f;
        for (int k = 0; k < rs.top; ++k) {
            const int slot = rs.slot_of[(size_t)blockIdx.x * rs.top + k];
            const float v = slot >= 0 ? rs.yp[(size_t)slot * D + c] : to_f<T>(hin[o + c]);
            acc = fmaf(rs.sel_w ? rs.sel_w[(size_t)blockIdx.x * rs.top + k] : 1.0f, v, acc);
        }
        return acc;
    };
    if (D <= (int)blockDim.x * kRowRegs) {
        // every operand is loaded before the first reduction: the kernel waits for global memory once
        float yv[kRowRegs], xv[kRowRegs], lv[kRowRegs], bv[kRowRegs], nv[kRowRegs];
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            const bool in = c < D;
            yv[i] = in ? y_at(c) : 0.0f;
            xv[i] = in ? x[o + c] : 0.0f;
            lv[i] = in ? ls[c] : 0.0f;
            bv[i] = in ? wb[c] : 0.0f;
            nv[i] = (in && wn) ? wn[c] : 0.0f;
            ss += yv[i] * yv[i];
        }
        ss = block_sum(ss, red);
        const float r = 1.0f / sqrtf(ss / (float)D + eps);
        float s2 = 0.0f;
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            const float v = xv[i] + lv[i] * (yv[i] * r * (woff + bv[i]));
            xv[i] = v;
            if (c < D) {
                x[o + c] = v;
                s2 += v * v;
            }
        }
        if (!wn) return;
        s2 = block_sum(s2, red);
        const float r2 = 1.0f / sqrtf(s2 / (float)D + eps);
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < D) hn[o + c] = from_f<T>(xv[i] * r2 * (woff + nv[i]));
        }
        return;
    }
    float ss = 0.0f;
    float* ysum = row;            // the sublayer's output of this row, then the new row
    for (int c = threadIdx.x; c < D; c += blockDim.x) { const float v = y_at(c); ysum[c] = v; ss += v * v; }
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)D + eps);
    float s2 = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = x[o + c] + ls[c] * (ysum[c] * r * (woff + wb[c]));
        x[o + c] = v;
        row[c] = v;
        s2 += v * v;
    }
    if (!wn) return;
    s2 = block_sum(s2, red);
    const float r2 = 1.0f / sqrtf(s2 / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) hn[o + c] = from_f<T>(row[c] * r2 * (woff + wn[c]));
}

// Three sums over the block at once; every thread gets the results.  `red` holds 3 x 33 floats.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*red)[33]) {
    a = warp_sum(a);
    b = warp_sum(b);
    c = warp_sum(c);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) { red[0][w] = a; red[1][w] = b; red[2][w] = c; }
    __syncthreads();
    if (w < 3) {
        float t = l < nw ? red[w][l] : 0.0f;
        t = warp_sum(t);
        if (l == 0) red[w][32] = t;
    }
    __syncthreads();
    a = red[0][32];
    b = red[1][32];
    c = red[2][32];
}

template <class T> __device__ __forceinline__ void store4(T* p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* p, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, float a, float b, float c, float d) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// PolyNorm: out = a z/rms(z) + b z^2/rms(z^2) + c z^3/rms(z^3) + e over a token's feed-forward vector.  The three sums
// are taken in one pass and reduced together; rows whose length is a multiple of 4 move as 16-byte pieces.
template <class T>
__global__ void polynorm_kernel(const float* __restrict__ z, const float* __restrict__ coef, float eps, int F, T* __restrict__ out) {
    __shared__ float red[3][33];
    const size_t o = (size_t)blockIdx.x * F;
    const bool vec = F % 4 == 0;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    auto add = [&](float v) {
        const float v2 = v * v;
        s2 += v2;
        s4 += v2 * v2;
        s6 += v2 * v2 * v2;
    };
    if (vec) {
        for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(z + o + c);
            add(v.x); add(v.y); add(v.z); add(v.w);
        }
    } else {
        for (int c = threadIdx.x; c < F; c += blockDim.x) add(z[o + c]);
    }
    block_sum3(s2, s4, s6, red);
    const float a = coef[0] / sqrtf(s2 / (float)F + eps), b = coef[1] / sqrtf(s4 / (float)F + eps),
                cc = coef[2] / sqrtf(s6 / (float)F + eps), e = coef[3];
    auto f = [&](float v) { return a * v + b * v * v + cc * v * v * v + e; };
    if (vec) {
        for (int c = threadIdx.x * 4; c < F; c += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(z + o + c);
            store4<T>(out + o + c, f(v.x), f(v.y), f(v.z), f(v.w));
        }
    } else {
        for (int c = threadIdx.x; c < F; c += blockDim.x) out[o + c] = from_f<T>(f(z[o + c]));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Where the operands of a matrix product live beyond the plain case (a [M, K], w [N, K], y [M, N], all contiguous).
//  - lda / ldy: row strides of a and y; blockIdx.z is a batch index with the strides sa / sw / sy (one product per head).
//  - grouped rows (tile_group != nullptr): the rows are sorted by group (expert), group g owning rows seg[g] .. seg[g+1]-1
//    and the weight matrix w + g * sw; blockIdx.y walks a tile table built on the device (tiles beyond *n_tiles leave at
//    once), and row r of the sorted order reads a's row gather[r] / gather_div (gather == nullptr: row r itself).
//  - bf16 products only: a_f32 -- a holds fp32 and is rounded to bf16 as it is staged; y_bf16 -- y holds bf16 (a result that
//    feeds the next product directly).
struct GemmIo {
    int lda, ldy;
    long long sa, sw, sy;
    const int32_t *tile_group, *tile_row0, *seg, *n_tiles, *gather;
    int gather_div;
    int a_f32, y_bf16;
};
constexpr int kGroupTile = 32;     // rows per tile of a grouped product (the tile table is built for this height)
static GemmIo plain_io(int K, int N) {
    GemmIo io;
    io.lda = K; io.ldy = N; io.sa = io.sw = io.sy = 0;
    io.tile_group = io.tile_row0 = io.seg = io.n_tiles = io.gather = nullptr;
    io.gather_div = 1;
    io.a_f32 = io.y_bf16 = 0;
    return io;
}

// Matrix product, fp32: y[M, N] = a[M, K] . w[N, K]^T with plain FMAs, k ascending (the result of a row does not depend on M).
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) gemm_f32_kernel(const float* __restrict__ a, const float* __restrict__ w,
                                                                        float* __restrict__ y, int M, int N, int K, const GemmIo io) {
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    __shared__ long long arow[BM];
    int m0 = blockIdx.y * BM;
    const int n0 = blockIdx.x * BN;
    a += blockIdx.z * io.sa;
    w += blockIdx.z * io.sw;
    y += blockIdx.z * io.sy;
    if (io.tile_group) {
        if ((int)blockIdx.y >= *io.n_tiles) return;
        const int g = io.tile_group[blockIdx.y];
        m0 = io.tile_row0[blockIdx.y];
        M = io.seg[g + 1];
        w += (long long)g * io.sw;
    }
    for (int r = threadIdx.x; r < BM; r += NT) {
        const int m = m0 + r;
        arow[r] = m < M ? (long long)(io.gather ? io.gather[m] / io.gather_div : m) * io.lda : -1;
    }
    __syncthreads();
    const int tx = threadIdx.x % (BN / TN), ty = threadIdx.x / (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += NT) {
            const int r = i / BK, c = i % BK;
            As[c][r] = (arow[r] >= 0 && k0 + c < K) ? a[arow[r] + k0 + c] : 0.0f;
        }
        for (int i = threadIdx.x; i < BN * BK; i += NT) {
            const int r = i / BK, c = i % BK;
            Ws[c][r] = (n0 + r < N && k0 + c < K) ? w[(size_t)(n0 + r) * K + k0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM], wv[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wv[j] = Ws[k][tx + j * (BN / TN)];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int m = m0 + ty * TM + i, n = n0 + tx + j * (BN / TN);
            if (m < M && n < N) y[(size_t)m * io.ldy + n] = acc[i][j];
        }
}

// Matrix product, bf16 inputs on the tensor cores (mma.sync m16n8k16, fp32 accumulation): 4 warps, tile (WR*MT*16) x (WC*NT*8),
// K in steps of 32 through shared memory, the next step's global loads in flight during the MMAs.
constexpr int kGemmBK = 32;
constexpr int kGemmLd = kGemmBK + 8;   // 80-byte rows: fragment loads hit 32 distinct banks

// off[i]: element offset of the i-th row this thread fetches (negative: a row outside the matrix, read as zeros)
template <int ROWS>
__device__ __forceinline__ void gemm_fetch(const bf16* __restrict__ src, const long long (&off)[ROWS * 4 / 128], int K, int k0, bool vec,
                                           uint4 (&reg)[ROWS * 4 / 128], bool f32 = false) {
#pragma unroll
    for (int i = 0; i < ROWS * 4 / 128; ++i) {
        const int c = (threadIdx.x & 3) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (off[i] >= 0 && f32) {
            const float* p = reinterpret_cast<const float*>(src) + off[i] + k0 + c;
            float e[8];
            if (vec && k0 + c + 8 <= K) {
                const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
                e[0] = lo.x; e[1] = lo.y; e[2] = lo.z; e[3] = lo.w; e[4] = hi.x; e[5] = hi.y; e[6] = hi.z; e[7] = hi.w;
            } else {
#pragma unroll
                for (int x = 0; x < 8; ++x) e[x] = (k0 + c + x < K) ? p[x] : 0.0f;
            }
            v = make_uint4(pack_bf16(e[0], e[1]), pack_bf16(e[2], e[3]), pack_bf16(e[4], e[5]), pack_bf16(e[6], e[7]));
        } else if (off[i] >= 0) {
            const bf16* p = src + off[i] + k0 + c;
            if (vec && k0 + c + 8 <= K) {
                v = *reinterpret_cast<const uint4*>(p);
            } else {
                uint16_t h[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = (k0 + c + e < K) ? reinterpret_cast<const uint16_t*>(p)[e] : (uint16_t)0;
                v.x = h[0] | ((uint32_t)h[1] << 16); v.y = h[2] | ((uint32_t)h[3] << 16);
                v.z = h[4] | ((uint32_t)h[5] << 16); v.w = h[6] | ((uint32_t)h[7] << 16);
            }
        }
        reg[i] = v;
    }
}
template <int ROWS>
__device__ __forceinline__ void gemm_stash(bf16* dst, const uint4 (&reg)[ROWS * 4 / 128]) {
#pragma unroll
    for (int i = 0; i < ROWS * 4 / 128; ++i) {
        const int id = threadIdx.x + i * 128, r = id >> 2, c = (id & 3) * 8;
        *reinterpret_cast<uint4*>(dst + r * kGemmLd + c) = reg[i];
    }
}

// `vec`: every row of a and w starts on a 16-byte boundary and K is a multiple of 8 (whole 16-byte pieces).
template <int WR, int WC, int MT, int NT>
__global__ void __launch_bounds__(128) gemm_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, float* __restrict__ y,
                                                        int M, int N, int K, const GemmIo io, const bool vec) {
    static_assert(WR * WC == 4, "four warps");
    constexpr int BM = WR * MT * 16, BN = WC * NT * 8;
    static_assert(BM % 32 == 0 && BN % 32 == 0, "tile rows are fetched 32 at a time");
    __shared__ __align__(16) bf16 As[2][BM * kGemmLd];
    __shared__ __align__(16) bf16 Ws[2][BN * kGemmLd];
    int m0 = blockIdx.y * BM;
    const int n0 = blockIdx.x * BN;
    const bool af = io.a_f32 != 0;
    a = af ? reinterpret_cast<const bf16*>(reinterpret_cast<const float*>(a) + blockIdx.z * io.sa) : a + blockIdx.z * io.sa;
    w += blockIdx.z * io.sw;
    const size_t y_base = (size_t)blockIdx.z * io.sy;
    if (io.tile_group) {
        if ((int)blockIdx.y >= *io.n_tiles) return;
        const int g = io.tile_group[blockIdx.y];
        m0 = io.tile_row0[blockIdx.y];
        M = io.seg[g + 1];
        w += (long long)g * io.sw;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int wm = (warp / WC) * MT * 16, wn = (warp % WC) * NT * 8;
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
    uint4 ra[BM * 4 / 128], rw[BN * 4 / 128];
    long long oa[BM * 4 / 128], ow[BN * 4 / 128];
#pragma unroll
    for (int i = 0; i < BM * 4 / 128; ++i) {
        const int m = m0 + ((threadIdx.x + i * 128) >> 2);
        oa[i] = m < M ? (long long)(io.gather ? io.gather[m] / io.gather_div : m) * io.lda : -1;
    }
#pragma unroll
    for (int i = 0; i < BN * 4 / 128; ++i) {
        const int n = n0 + ((threadIdx.x + i * 128) >> 2);
        ow[i] = n < N ? (long long)n * K : -1;
    }
    gemm_fetch<BM>(a, oa, K, 0, vec, ra, af);
    gemm_fetch<BN>(w, ow, K, 0, vec, rw);
    gemm_stash<BM>(As[0], ra);
    gemm_stash<BN>(Ws[0], rw);
    __syncthreads();
    const int steps = (K + kGemmBK - 1) / kGemmBK;
    for (int s = 0; s < steps; ++s) {
        const int cur = s & 1;
        if (s + 1 < steps) {
            gemm_fetch<BM>(a, oa, K, (s + 1) * kGemmBK, vec, ra, af);
            gemm_fetch<BN>(w, ow, K, (s + 1) * kGemmBK, vec, rw);
        }
#pragma unroll
        for (int kk = 0; kk < kGemmBK; kk += 16) {
            uint32_t af[MT][4], bfr[NT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                const bf16* p = As[cur] + (wm + i * 16 + g) * kGemmLd + kk + tq * 2;
                af[i][0] = *reinterpret_cast<const uint32_t*>(p);
                af[i][1] = *reinterpret_cast<const uint32_t*>(p + 8 * kGemmLd);
                af[i][2] = *reinterpret_cast<const uint32_t*>(p + 8);
                af[i][3] = *reinterpret_cast<const uint32_t*>(p + 8 * kGemmLd + 8);
            }
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const bf16* p = Ws[cur] + (wn + j * 8 + g) * kGemmLd + kk + tq * 2;
                bfr[j][0] = *reinterpret_cast<const uint32_t*>(p);
                bfr[j][1] = *reinterpret_cast<const uint32_t*>(p + 8);
            }
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_bf16_16816(acc[i][j], af[i][0], af[i][1], af[i][2], af[i][3], bfr[j][0], bfr[j][1]);
        }
        if (s + 1 < steps) {
            gemm_stash<BM>(As[cur ^ 1], ra);
            gemm_stash<BN>(Ws[cur ^ 1], rw);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int m = m0 + wm + i * 16 + g, n = n0 + wn + j * 8 + tq * 2;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int mm = m + (e >> 1) * 8, nn = n + (e & 1);
                if (mm < M && nn < N) {
                    const size_t at = y_base + (size_t)mm * io.ldy + nn;
                    if (io.y_bf16) reinterpret_cast<bf16*>(y)[at] = __float2bfloat16_rn(acc[i][j][e]);
                    else y[at] = acc[i][j][e];
                }
            }
        }
}

// Matrix product for very few rows (decoding): WPC warps per output column (each a 1/WPC interleaved share of K, the
// shares added in a fixed order), lanes cut K into 16-byte pieces; the weights are streamed once, the MR activation
// rows come from L1/L2.  WPC follows from N alone (narrow products get more warps per column so that the grid still
// covers the SMs).  Needs K % 8 == 0 and 16-byte aligned operands.
template <int MR, int WPC>
__global__ void __launch_bounds__(256) gemv_bf16_kernel(const bf16* __restrict__ a, const bf16* __restrict__ w, float* __restrict__ y,
                                                        int M, int N, int K) {
    __shared__ float part[8][MR];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, kw = warp % WPC;
    const int n = blockIdx.x * (8 / WPC) + warp / WPC;
    const bool valid = n < N;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.0f;
    if (valid) {
        const bf16* wr = w + (size_t)n * K;
        for (int k = (kw * 32 + lane) * 8; k < K; k += 256 * WPC) {
            const uint4 wv = ldg_stream(wr + k);
            const float w0 = bf_lo(wv.x), w1 = bf_hi(wv.x), w2 = bf_lo(wv.y), w3 = bf_hi(wv.y), w4 = bf_lo(wv.z), w5 = bf_hi(wv.z),
                        w6 = bf_lo(wv.w), w7 = bf_hi(wv.w);
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                if (m < M) {
                    const uint4 av = ldg_v4(a + (size_t)m * K + k);
                    float t = acc[m];
                    t = fmaf(bf_lo(av.x), w0, t); t = fmaf(bf_hi(av.x), w1, t); t = fmaf(bf_lo(av.y), w2, t); t = fmaf(bf_hi(av.y), w3, t);
                    t = fmaf(bf_lo(av.z), w4, t); t = fmaf(bf_hi(av.z), w5, t); t = fmaf(bf_lo(av.w), w6, t); t = fmaf(bf_hi(av.w), w7, t);
                    acc[m] = t;
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        const float t = warp_sum(acc[m]);
        if (WPC == 1) {
            if (lane == 0 && valid && m < M) y[(size_t)m * N + n] = t;
        } else if (lane == 0) {
            part[warp][m] = t;
        }
    }
    if (WPC > 1) {
        __syncthreads();
        if (kw == 0 && lane < MR && lane < M && valid) {
            float t = part[warp][lane];
#pragma unroll
            for (int x = 1; x < WPC; ++x) t += part[warp + x][lane];
            y[(size_t)lane * N + n] = t;
        }
    }
}

// Matrix product for many rows (prompt portions), bf16 on the 5th-generation tensor cores: the library's tcgen05 tile
// (umma.cuh: TMA loads into a 128-byte-swizzled ring, accumulators in tensor memory) over 128 rows x kTcTileN columns,
// one persistent CTA per SM walking the tiles; row tiles that share a weight tile run on neighbouring CTAs.  Rows and
// columns outside the matrices are zero-filled by TMA (a partial last K stage adds zeros); rows past M of the activation
// buffer hold stale values whose accumulator lanes are never stored.
constexpr int kTcTileN = umma::kMaxN;
constexpr int kTcThreads = 512;
constexpr int kTcSmemBytes = umma::kRingBytes + 1024;
constexpr int kTcMinRows = 257;          // below this the mma.sync tiles fill the GPU better than 128-row tiles

// Grouped rows (io.tile_group != nullptr): the row tiles come from the device-built table (128 rows each, group g's rows end
// at seg[g + 1]; rows of the tile beyond that belong to the next group and are computed but not stored), and group g's
// weights are rows g * N .. of the weight map.
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
                                                                float* __restrict__ y, int M, int N, int K, const GemmIo io) {
    extern __shared__ unsigned char tc_smem[];
    __shared__ umma::Bars bars;
    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem) + 1023) & ~(uintptr_t)1023);
    umma::Pipe pipe;
    umma::setup(&bars, pipe, (uint32_t)umma::kAcc, 2u);
    const int m_tiles = io.tile_group ? *io.n_tiles : (M + umma::kM - 1) / umma::kM, n_tiles = (N + kTcTileN - 1) / kTcTileN;
    const int k_pad = (K + umma::kBK - 1) / umma::kBK * umma::kBK;
    const bool vec = N % 4 == 0;
    for (int u = blockIdx.x; u < m_tiles * n_tiles; u += gridDim.x) {
        int m0 = (u % m_tiles) * umma::kM, w_row = 0;
        const int n0 = (u / m_tiles) * kTcTileN;
        if (io.tile_group) {
            const int g = io.tile_group[u % m_tiles];
            m0 = io.tile_row0[u % m_tiles];
            M = io.seg[g + 1];
            w_row = g * N;
        }
        umma::BSrc b0, b1;
        b0.tm = &tm_w; b0.row0 = w_row + n0; b0.n = kTcTileN; b0.box = kTcTileN;
        b1.tm = nullptr; b1.row0 = 0; b1.n = 0; b1.box = kTcTileN;
        umma::tile_mma_tma<kTcThreads>(ring, &bars, pipe, k_pad, &tm_a, m0, b0, b1);
        umma::tile_epilogue(&bars, kTcTileN, [&](int row, int c0, const float (&acc)[8]) {
            const int m = m0 + row, n = n0 + c0;
            if (m >= M || n >= N) return;
            float* out = y + (size_t)m * N + n;
            if (vec && n + 8 <= N) {
                *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<float4*>(out + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    if (n + e < N) out[e] = acc[e];
            }
        }, kTcTileN);
    }
    umma::teardown(&bars);
}

// ---------------------------------------------------------------------------------------------------------------------
// Softmax attention over the paged pool.  A cached position holds, per key/value head, a key row of d elements (row
// stride k_ld) and a value row of dv elements (row stride v_ld); with v_in_k the value is the first dv elements of the key
// row (a latent that serves as both).  Optional per head: a distance penalty r1 ln(1 + r2 (i - j)) taken off the score
// (r1 == nullptr: none) and a key-less sink logit in the softmax denominator (sink == nullptr: none).  The output is
// multiplied by sigmoid(proj[t][gate_off + h * gate_ld + c * gate_step]): a gate per channel or (gate_step 0) per head.
// Sink attention's proj row layout: q [H*d] | k [G*d] | v [G*dv] | gate [H*dv] (no gate rows with has_gate == 0).
// Further options, each off at its zero value: `bias` added to the projection's rows as they are read; `window` > 0 limits
// a query at position i to the keys 0 <= i - j < window; `softcap` > 0 bends the scaled score to softcap * tanh(score /
// softcap) before the penalties; `slope` takes slope_h * (i - j) off.  The result is multiplied by out_scale and written
// with the row stride out_ld (two mixers side by side share one buffer).
struct AttnArgs {
    const float* proj;
    int n_in;
    const int32_t *tok_seq, *tok_pos, *block_table;
    int max_pages, page_size, n_pages;
    size_t page_elems, k_off, v_off;   // element offsets of this run's keys / values inside a page
    int k_ld, v_ld, v_in_k;
    size_t gate_off;
    int gate_ld, gate_step;
    int H, G, d, dv;
    float scale, eps;
    const float *q_norm, *k_norm, *r1, *r2, *sink;
    int n_tokens;
    int32_t* err;
    const int32_t* seq_start;
    int split_len, n_splits, short_rows;   // few-token path: key range per block, ranges per row, rows = sequences x kShortSeq
    float* part;                           // [short_rows][H][n_splits][dv + 2]: running maximum, denominator, unnormalised output
    const float *bias, *slope;
    int window, has_gate, out_ld;
    float softcap, two_over_cap, out_scale;      // two_over_cap = 2 / softcap (0 without a cap)
};

// first key a query at `pos` sees
__device__ __forceinline__ int attn_first_key(const AttnArgs& A, int pos) { return A.window > 0 ? max(0, pos - A.window + 1) : 0; }

// what follows the dot product: scale, soft cap, distance penalties.  FAST: hardware exponential / logarithm (bf16 engine).
template <bool FAST>
__device__ __forceinline__ float attn_score(const AttnArgs& A, float dot, int dist, float r1, float r2, float slope) {
    float s = dot * A.scale;
    if (A.softcap > 0.0f) {
        // FAST: tanh z = 1 - 2 / (e^{2z} + 1) with the hardware exponential and division (an overflowing e^{2z} gives 1)
        if (FAST) s = A.softcap * (1.0f - __fdividef(2.0f, __expf(s * A.two_over_cap) + 1.0f));
        else s = A.softcap * tanhf(s / A.softcap);
    }
    if (A.r1) s -= r1 * (FAST ? __logf(1.0f + r2 * (float)dist) : log1pf(r2 * (float)dist));
    if (A.slope) s -= slope * (float)dist;
    return s;
}

// One warp per (token, slot): slots 0..H-1 norm a query head into qbuf, H..H+G-1 norm a key head into the pool,
// H+G..H+2G-1 copy a value head into the pool.
template <class T>
__global__ void attn_prep_kernel(const AttnArgs A, T* __restrict__ qbuf, T* __restrict__ pool) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int slots = A.H + 2 * A.G;
    if (unit >= A.n_tokens * slots) return;
    const int t = unit / slots, s = unit % slots;
    const float* row = A.proj + (size_t)t * A.n_in;
    if (s < A.H) {
        const float* q = row + s * A.d;
        const float* qb = A.bias ? A.bias + s * A.d : nullptr;
        float ss = 0.0f;
        for (int c = lane; c < A.d; c += 32) { const float v = q[c] + (qb ? qb[c] : 0.0f); ss += v * v; }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)A.d + A.eps);
        for (int c = lane; c < A.d; c += 32) qbuf[((size_t)t * A.H + s) * A.d + c] = from_f<T>((q[c] + (qb ? qb[c] : 0.0f)) * r * A.q_norm[c]);
        return;
    }
    const int pos = A.tok_pos[t];
    const int pg = pos / A.page_size, in_pg = pos % A.page_size;
    int page = pg < A.max_pages ? A.block_table[(size_t)A.tok_seq[t] * A.max_pages + pg] : -1;
    if (page < 0 || page >= A.n_pages) {
        if (lane == 0) atomicExch(A.err, 1);
        return;
    }
    T* base = pool + (size_t)page * A.page_elems;
    if (s < A.H + A.G) {
        const int gk = s - A.H;
        const float* k = row + A.H * A.d + gk * A.d;
        const float* kb = A.bias ? A.bias + A.H * A.d + gk * A.d : nullptr;
        float ss = 0.0f;
        for (int c = lane; c < A.d; c += 32) { const float v = k[c] + (kb ? kb[c] : 0.0f); ss += v * v; }
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)A.d + A.eps);
        T* dst = base + A.k_off + ((size_t)gk * A.page_size + in_pg) * A.d;
        for (int c = lane; c < A.d; c += 32) dst[c] = from_f<T>((k[c] + (kb ? kb[c] : 0.0f)) * r * A.k_norm[c]);
    } else {
        const int gv = s - A.H - A.G;
        const float* v = row + (A.H + A.G) * A.d + gv * A.dv;
        const float* vb = A.bias ? A.bias + (A.H + A.G) * A.d + gv * A.dv : nullptr;
        T* dst = base + A.v_off + ((size_t)gv * A.page_size + in_pg) * A.dv;
        for (int c = lane; c < A.dv; c += 32) dst[c] = from_f<T>(v[c] + (vb ? vb[c] : 0.0f));
    }
}

// The same preparation with query and key norms over the WHOLE projection: one root mean square for all query heads of a
// token (weights q_norm [H*d]) and one for all key heads (k_norm [G*d]).  One block per token.  Loads go out kPrepBatch
// at a time before their first use: a lone token (decoding) waits for memory a few times, not once per element.
constexpr int kPrepBatch = 4;

template <class T>
__global__ void __launch_bounds__(256) attn_prep_whole_kernel(const AttnArgs A, T* __restrict__ qbuf, T* __restrict__ pool) {
    __shared__ float red[2][33];
    const int t = blockIdx.x, nq = A.H * A.d, nk = A.G * A.d, nv = A.G * A.dv;
    const float* row = A.proj + (size_t)t * A.n_in;
    const int pos = A.tok_pos[t];
    const int pg = pos / A.page_size, in_pg = pos % A.page_size;
    const int page = pg < A.max_pages ? A.block_table[(size_t)A.tok_seq[t] * A.max_pages + pg] : -1;
    // sum of squares of row[lo .. lo + n) + bias
    auto sum_sq = [&](int lo, int n) {
        float ss = 0.0f;
        for (int c0 = threadIdx.x; c0 < n; c0 += blockDim.x * kPrepBatch) {
            float v[kPrepBatch], bv[kPrepBatch];
#pragma unroll
            for (int u = 0; u < kPrepBatch; ++u) {
                const int c = c0 + u * blockDim.x;
                v[u] = c < n ? row[lo + c] : 0.0f;
                bv[u] = (c < n && A.bias) ? A.bias[lo + c] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < kPrepBatch; ++u) ss = fmaf(v[u] + bv[u], v[u] + bv[u], ss);
        }
        return ss;
    };
    float sq = sum_sq(0, nq), sk = sum_sq(nq, nk);
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) { red[0][w] = sq; red[1][w] = sk; }
    __syncthreads();
    sq = 0.0f;
    sk = 0.0f;
    for (int i = 0; i < nw; ++i) { sq += red[0][i]; sk += red[1][i]; }      // the same order in every thread
    const float rq = 1.0f / sqrtf(sq / (float)nq + A.eps), rk = 1.0f / sqrtf(sk / (float)nk + A.eps);
    // element c of row[lo ..) + bias, times mul, times weight[c] (nullptr: 1) -> store(c, value)
    auto emit = [&](int lo, int n, float mul, const float* weight, auto store) {
        for (int c0 = threadIdx.x; c0 < n; c0 += blockDim.x * kPrepBatch) {
            float v[kPrepBatch], wv[kPrepBatch];
#pragma unroll
            for (int u = 0; u < kPrepBatch; ++u) {
                const int c = c0 + u * blockDim.x;
                v[u] = c < n ? row[lo + c] + (A.bias ? A.bias[lo + c] : 0.0f) : 0.0f;
                wv[u] = (c < n && weight) ? weight[c] : 1.0f;
            }
#pragma unroll
            for (int u = 0; u < kPrepBatch; ++u) {
                const int c = c0 + u * blockDim.x;
                if (c < n) store(c, v[u] * mul * wv[u]);
            }
        }
    };
    emit(0, nq, rq, A.q_norm, [&](int c, float v) { qbuf[(size_t)t * nq + c] = from_f<T>(v); });
    if (page < 0 || page >= A.n_pages) {
        if (threadIdx.x == 0) atomicExch(A.err, 1);
        return;
    }
    T* base = pool + (size_t)page * A.page_elems;
    emit(nq, nk, rk, A.k_norm, [&](int c, float v) {
        const int g = c / A.d, i = c - g * A.d;
        base[A.k_off + ((size_t)g * A.page_size + in_pg) * A.d + i] = from_f<T>(v);
    });
    emit(nq + nk, nv, 1.0f, nullptr, [&](int c, float v) {
        const int g = c / A.dv, i = c - g * A.dv;
        base[A.v_off + ((size_t)g * A.page_size + in_pg) * A.dv + i] = from_f<T>(v);
    });
}

// One warp per (token, query head), 32 keys per round: lane j scores key j (full dot product, the query in shared
// memory), the round's softmax weights are shared by shuffles and every lane accumulates dv / 32 output columns.
// The sink enters as the initial state of the running softmax: maximum = sink, denominator = 1, no value.
constexpr int kAttnWarps = 4;
constexpr int kAttnMaxV = 16;  // value size up to 512; the kernels are built for 8 (up to 256) and 16 lanes' worth of columns

__device__ __forceinline__ float attn_gate(const AttnArgs& A, size_t t, int h, int c) {
    if (!A.has_gate) return A.out_scale;
    return A.out_scale * sigmoidf_(A.proj[t * A.n_in + A.gate_off + (size_t)h * A.gate_ld + (size_t)c * A.gate_step]);
}

template <class T, int MAXV>
__global__ void __launch_bounds__(kAttnWarps * 32) attn_kernel(const AttnArgs A, const T* __restrict__ qbuf, const T* __restrict__ pool,
                                                               T* __restrict__ out) {
    extern __shared__ float qs_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int unit = blockIdx.x * kAttnWarps + warp;
    if (unit >= A.n_tokens * A.H) return;
    const int t = unit / A.H, h = unit % A.H;
    const int g = h / (A.H / A.G);
    float* qs = qs_all + warp * A.d;
    for (int c = lane; c < A.d; c += 32) qs[c] = to_f<T>(qbuf[((size_t)t * A.H + h) * A.d + c]);
    __syncwarp();
    const int pos = A.tok_pos[t];
    const int32_t* bt = A.block_table + (size_t)A.tok_seq[t] * A.max_pages;
    const float r1 = A.r1 ? A.r1[h] : 0.0f, r2 = A.r1 ? A.r2[h] : 0.0f, slope = A.slope ? A.slope[h] : 0.0f;
    float m = A.sink ? A.sink[h] : -INFINITY, l = A.sink ? 1.0f : 0.0f;
    float o[MAXV];
#pragma unroll
    for (int e = 0; e < MAXV; ++e) o[e] = 0.0f;
    for (int j0 = attn_first_key(A, pos); j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        const T* vrow = nullptr;
        if (j <= pos) {
            const int page = bt[j / A.page_size], in_pg = j % A.page_size;
            const T* base = pool + (size_t)page * A.page_elems;
            const T* k = base + A.k_off + ((size_t)g * A.page_size + in_pg) * A.k_ld;
            vrow = base + A.v_off + ((size_t)g * A.page_size + in_pg) * A.v_ld;
            float dot = 0.0f;
            for (int c = 0; c < A.d; ++c) dot = fmaf(qs[c], to_f<T>(k[c]), dot);
            s = attn_score<false>(A, dot, pos - j, r1, r2, slope);
        }
        const float mn = fmaxf(m, warp_max(s));          // finite: lane 0 of every round holds a visible key
        const float p = (j <= pos) ? expf(s - mn) : 0.0f;
        const float corr = expf(m - mn);
        l = l * corr + warp_sum(p);
        m = mn;
#pragma unroll
        for (int e = 0; e < MAXV; ++e) o[e] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const T* vr = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(vrow), jj));
#pragma unroll
            for (int e = 0; e < MAXV; ++e) {
                const int c = lane + e * 32;
                if (c < A.dv) o[e] = fmaf(pj, to_f<T>(vr[c]), o[e]);
            }
        }
    }
    const float inv = 1.0f / l;
#pragma unroll
    for (int e = 0; e < MAXV; ++e) {
        const int c = lane + e * 32;
        if (c < A.dv) out[(size_t)t * A.out_ld + h * A.dv + c] = from_f<T>(o[e] * inv * attn_gate(A, t, h, c));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention for sequences that bring few tokens (decoding, short portions): the keys of a row are cut into fixed
// ranges of A.split_len positions, one block per (row, key/value head, range), whose warps take the query heads of
// that key/value head; a second kernel merges the ranges with the sink and applies the gate.  The ranges are absolute
// positions, so a row's result does not depend on what else is in the step.
constexpr int kGraphMaxTokens = 64;   // steps of at most this many tokens are replayed from a captured graph
constexpr int kShortSeq = 8;          // a sequence with at most this many tokens in a step takes this path

// q (fp32, shared memory) . k (one cached key row), 16-byte loads where the row allows them
template <class T> __device__ __forceinline__ float key_dot(const float* qs, const T* k, int d);
template <> __device__ __forceinline__ float key_dot<float>(const float* qs, const float* k, int d) {
    float dot = 0.0f;
    if (d % 4 == 0 && reinterpret_cast<uintptr_t>(k) % 16 == 0) {
        for (int c = 0; c < d; c += 4) {
            const float4 v = *reinterpret_cast<const float4*>(k + c);
            dot = fmaf(qs[c], v.x, dot); dot = fmaf(qs[c + 1], v.y, dot); dot = fmaf(qs[c + 2], v.z, dot); dot = fmaf(qs[c + 3], v.w, dot);
        }
    } else {
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], k[c], dot);
    }
    return dot;
}
template <> __device__ __forceinline__ float key_dot<bf16>(const float* qs, const bf16* k, int d) {
    float dot = 0.0f;
    if (d % 8 == 0 && reinterpret_cast<uintptr_t>(k) % 16 == 0) {
        for (int c = 0; c < d; c += 8) {
            const uint4 v = ldg_v4(k + c);
            dot = fmaf(qs[c], bf_lo(v.x), dot); dot = fmaf(qs[c + 1], bf_hi(v.x), dot);
            dot = fmaf(qs[c + 2], bf_lo(v.y), dot); dot = fmaf(qs[c + 3], bf_hi(v.y), dot);
            dot = fmaf(qs[c + 4], bf_lo(v.z), dot); dot = fmaf(qs[c + 5], bf_hi(v.z), dot);
            dot = fmaf(qs[c + 6], bf_lo(v.w), dot); dot = fmaf(qs[c + 7], bf_hi(v.w), dot);
        }
    } else {
        for (int c = 0; c < d; ++c) dot = fmaf(qs[c], __bfloat162float(k[c]), dot);
    }
    return dot;
}

template <class T, int MAXV>
__global__ void __launch_bounds__(256) attn_split_kernel(const AttnArgs A, const T* __restrict__ qbuf, const T* __restrict__ pool) {
    // One block per (row, key/value head x group of up to 8 of its query heads, key range); one warp per query head.
    // 32 keys and values at a time are staged in shared memory (rows padded by 16 bytes: conflict-free row-per-lane
    // reads), so that no global load sits inside the softmax / value loops.
    extern __shared__ __align__(16) unsigned char sm_raw[];
    constexpr int kPad = 16 / (int)sizeof(T);
    const int s = blockIdx.x / kShortSeq, r = blockIdx.x % kShortSeq;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    if (n > kShortSeq || r >= n) return;
    const int t = t0 + r, pos = A.tok_pos[t];
    // with a window the ranges are counted from the one that holds the row's first visible key
    const int j_first = attn_first_key(A, pos);
    const int range = j_first / A.split_len + blockIdx.z;
    if (range * A.split_len > pos) return;
    const int j_lo = max(range * A.split_len, j_first);
    const int j_hi = min(pos, (range + 1) * A.split_len - 1);
    const int Gq = A.H / A.G, nwarp = blockDim.x >> 5;
    const int groups = (Gq + nwarp - 1) / nwarp;
    const int g = blockIdx.y / groups, hq = (blockIdx.y % groups) * nwarp + (threadIdx.x >> 5);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool active = hq < Gq;
    const int h = g * Gq + (active ? hq : 0);
    const int ldk = A.d + kPad, ldv = A.v_in_k ? ldk : A.dv + kPad;
    float* qs = reinterpret_cast<float*>(sm_raw) + warp * A.d;
    float* ps = reinterpret_cast<float*>(sm_raw) + nwarp * A.d + warp * 32;
    T* Ks = reinterpret_cast<T*>(sm_raw + (((size_t)nwarp * (A.d + 32) * 4 + 15) / 16) * 16);
    T* Vs = A.v_in_k ? Ks : Ks + 32 * ldk;
    const int32_t* bt = A.block_table + (size_t)s * A.max_pages;
    for (int c = lane; c < A.d; c += 32) qs[c] = to_f<T>(qbuf[((size_t)t * A.H + h) * A.d + c]);
    const float r1 = A.r1 ? A.r1[h] : 0.0f, r2 = A.r1 ? A.r2[h] : 0.0f, slope = A.slope ? A.slope[h] : 0.0f;
    float m = -INFINITY, l = 0.0f;
    float o[MAXV];
#pragma unroll
    for (int e = 0; e < MAXV; ++e) o[e] = 0.0f;
    // whole 16-byte pieces when every cached row starts on a 16-byte boundary (pages are 16-byte aligned)
    const bool kvec = (A.d * sizeof(T)) % 16 == 0 && (A.k_ld * sizeof(T)) % 16 == 0 && (A.k_off * sizeof(T)) % 16 == 0;
    const bool vvec = (A.dv * sizeof(T)) % 16 == 0 && (A.v_ld * sizeof(T)) % 16 == 0 && (A.v_off * sizeof(T)) % 16 == 0;
    const int kchunks = kvec ? A.d / kPad : A.d, vchunks = A.v_in_k ? 0 : (vvec ? A.dv / kPad : A.dv);
    for (int j0 = j_lo; j0 <= j_hi; j0 += 32) {
        const int cnt = min(32, j_hi - j0 + 1);
        __syncthreads();
        for (int idx = threadIdx.x; idx < cnt * (kchunks + vchunks); idx += blockDim.x) {
            const int row = idx / (kchunks + vchunks), c = idx % (kchunks + vchunks);
            const int j = j0 + row;
            const T* base = pool + (size_t)bt[j / A.page_size] * A.page_elems;
            const size_t in_pg = (size_t)g * A.page_size + j % A.page_size;
            if (c < kchunks) {
                const T* src = base + A.k_off + in_pg * A.k_ld;
                if (kvec) *reinterpret_cast<uint4*>(Ks + row * ldk + c * kPad) = *reinterpret_cast<const uint4*>(src + c * kPad);
                else Ks[row * ldk + c] = src[c];
            } else {
                const int cv = c - kchunks;
                const T* src = base + A.v_off + in_pg * A.v_ld;
                if (vvec) *reinterpret_cast<uint4*>(Vs + row * ldv + cv * kPad) = *reinterpret_cast<const uint4*>(src + cv * kPad);
                else Vs[row * ldv + cv] = src[cv];
            }
        }
        __syncthreads();
        if (!active) continue;
        const int j = j0 + lane;
        float sc = -INFINITY;
        if (lane < cnt) {
            sc = attn_score<false>(A, key_dot<T>(qs, Ks + lane * ldk, A.d), pos - j, r1, r2, slope);
        }
        const float mn = fmaxf(m, warp_max(sc));          // finite: lane 0 of every round holds a valid key
        const float p = lane < cnt ? expf(sc - mn) : 0.0f;
        const float corr = expf(m - mn);
        l = l * corr + warp_sum(p);
        m = mn;
        ps[lane] = p;
        __syncwarp();
#pragma unroll
        for (int e = 0; e < MAXV; ++e) o[e] *= corr;
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = ps[jj];
#pragma unroll
            for (int e = 0; e < MAXV; ++e) {
                const int c = lane + e * 32;
                if (c < A.dv) o[e] = fmaf(pj, to_f<T>(Vs[jj * ldv + c]), o[e]);
            }
        }
        __syncwarp();
    }
    if (!active) return;
    float* dst = A.part + (((size_t)blockIdx.x * A.H + h) * A.n_splits + blockIdx.z) * (A.dv + 2);
    if (lane == 0) { dst[0] = m; dst[1] = l; }
#pragma unroll
    for (int e = 0; e < MAXV; ++e) {
        const int c = lane + e * 32;
        if (c < A.dv) dst[2 + c] = o[e];
    }
}

// One warp per (row, query head): merges the ranges; the sink enters here, once, with no value.
template <class T, int MAXV>
__global__ void __launch_bounds__(128) attn_merge_kernel(const AttnArgs A, T* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= A.short_rows * A.H) return;
    const int x = unit / A.H, h = unit % A.H;
    const int s = x / kShortSeq, r = x % kShortSeq;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    if (n > kShortSeq || r >= n) return;
    const int t = t0 + r, pos = A.tok_pos[t];
    const int ns = pos / A.split_len - attn_first_key(A, pos) / A.split_len + 1;
    const float* src = A.part + ((size_t)x * A.H + h) * A.n_splits * (A.dv + 2);
    // lanes take the ranges' maxima and weights side by side; the value columns are then summed range by range with the
    // weights handed on by shuffles, so that no load waits for an earlier one
    const float sink = A.sink ? A.sink[h] : -INFINITY;
    float M = sink;
    for (int z = lane; z < ns; z += 32) M = fmaxf(M, src[(size_t)z * (A.dv + 2)]);
    M = warp_max(M);
    float l = 0.0f;
    float o[MAXV];
#pragma unroll
    for (int e = 0; e < MAXV; ++e) o[e] = 0.0f;
    for (int z0 = 0; z0 < ns; z0 += 32) {
        const int z = z0 + lane, cnt = min(32, ns - z0);
        float wz = 0.0f;
        if (z < ns) {
            const float* p = src + (size_t)z * (A.dv + 2);
            wz = expf(p[0] - M);
            l = fmaf(p[1], wz, l);
        }
#pragma unroll 4
        for (int i = 0; i < cnt; ++i) {
            const float w = __shfl_sync(0xffffffffu, wz, i);
            const float* p = src + (size_t)(z0 + i) * (A.dv + 2) + 2;
#pragma unroll
            for (int e = 0; e < MAXV; ++e) {
                const int c = lane + e * 32;
                if (c < A.dv) o[e] = fmaf(p[c], w, o[e]);
            }
        }
    }
    l = warp_sum(l) + expf(sink - M);
    const float inv = 1.0f / l;
#pragma unroll
    for (int e = 0; e < MAXV; ++e) {
        const int c = lane + e * 32;
        if (c < A.dv) out[(size_t)t * A.out_ld + h * A.dv + c] = from_f<T>(o[e] * inv * attn_gate(A, t, h, c));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Attention for prompt portions, bf16, on the tensor cores (mma.sync m16n8k16, fp32 accumulation).  One block per
// (64-row tile of a sequence's rows in this step, sequence, query head); each of the four warps owns 16 rows.  Keys and
// values are staged 64 positions at a time from the paged pool into shared memory (head sizes padded with zeros to DP).
// Scores, the distance penalty, the running maximum and the softmax weights are fp32; for the weights x values product a
// weight is split into a bf16 head and a bf16 remainder (two MMAs), which keeps 16 mantissa bits of it.  The sink is
// the initial state of the running softmax: maximum = sink, denominator = 1.
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(a));
}

// rows x cols bf16 from `src(row)` (nullptr: a row of zeros) into dst[row * LD + col], columns cols .. DP-1 zeroed.
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// 64 rows of `cols` bf16 into a [64][DP + 8] tile; src(row) is the row's address or nullptr (zero row).  ASYNC: whole
// 16-byte pieces of aligned rows go by cp.async (the caller commits and waits); everything else is stored directly.
template <int DP, bool ASYNC, class RowPtr>
__device__ __forceinline__ void stage_rows(bf16* dst, int cols, RowPtr src) {
    constexpr int LD = DP + 8;
    const bool vec = (cols % 8) == 0;
    for (int idx = threadIdx.x; idx < 64 * (DP / 8); idx += 128) {
        const int row = idx / (DP / 8), c = (idx % (DP / 8)) * 8;
        const bf16* p = src(row);
        uint4 v = make_uint4(0, 0, 0, 0);
        if (p && c < cols) {
            if (vec && (reinterpret_cast<uintptr_t>(p) % 16) == 0) {
                if (ASYNC) {
                    cp_async16(dst + row * LD + c, p + c);
                    continue;
                }
                v = *reinterpret_cast<const uint4*>(p + c);
            } else {
                uint16_t hh[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) hh[e] = (c + e < cols) ? reinterpret_cast<const uint16_t*>(p)[c + e] : (uint16_t)0;
                v.x = hh[0] | ((uint32_t)hh[1] << 16); v.y = hh[2] | ((uint32_t)hh[3] << 16);
                v.z = hh[4] | ((uint32_t)hh[5] << 16); v.w = hh[6] | ((uint32_t)hh[7] << 16);
            }
        }
        *reinterpret_cast<uint4*>(dst + row * LD + c) = v;
    }
}

// The exponentials and the penalty's logarithm use the hardware approximations (relative error about 2^-22): this form
// serves bf16 only, whose products carry 2^-9.
// DK / DV: key and value sizes padded to multiples of 16.  VK: the values are the first columns of the key rows (a cached
// latent that serves as both), so only key tiles are staged and DV <= DK.
template <int DK, int DV, bool VK>
__global__ void __launch_bounds__(128) attn_flash_kernel(const AttnArgs A, const bf16* __restrict__ qbuf, const bf16* __restrict__ pool,
                                                         bf16* __restrict__ out) {
    constexpr int LD = DK + 8, kTile = 64 * LD, LDV = VK ? LD : DV + 8, kTileV = 64 * LDV;
    static_assert(!VK || DV <= DK, "values inside the key rows");
    extern __shared__ __align__(16) unsigned char flash_smem[];      // keys [2][64][LD], values [2][64][LDV]: two tiles in turn
    bf16* Ks = reinterpret_cast<bf16*>(flash_smem);
    bf16* Vs = VK ? Ks : Ks + 2 * kTile;
    const int s = blockIdx.y;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    const int tile = gridDim.x - 1 - blockIdx.x;      // the tiles with the most keys start first
    if (n <= kShortSeq || tile * 64 >= n) return;
    const int h = blockIdx.z, g = h / (A.H / A.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
    const int pos0 = A.tok_pos[t0];
    const int32_t* bt = A.block_table + (size_t)s * A.max_pages;
    // queries of the tile -> A fragments
    stage_rows<DK, false>(Ks, A.d, [&](int row) -> const bf16* {
        return tile * 64 + row < n ? qbuf + ((size_t)(t0 + tile * 64 + row) * A.H + h) * A.d : nullptr;
    });
    __syncthreads();
    uint32_t qf[DK / 16][4];
#pragma unroll
    for (int kk = 0; kk < DK / 16; ++kk) {
        const bf16* p = Ks + (warp * 16 + gq) * LD + kk * 16 + tq * 2;
        qf[kk][0] = *reinterpret_cast<const uint32_t*>(p);
        qf[kk][1] = *reinterpret_cast<const uint32_t*>(p + 8 * LD);
        qf[kk][2] = *reinterpret_cast<const uint32_t*>(p + 8);
        qf[kk][3] = *reinterpret_cast<const uint32_t*>(p + 8 * LD + 8);
    }
    __syncthreads();
    const int row_a = tile * 64 + warp * 16 + gq, row_b = row_a + 8;
    const int i_a = pos0 + row_a, i_b = pos0 + row_b;
    const int last_pos = pos0 + min(n, tile * 64 + 64) - 1;
    const bool penalty = A.r1 != nullptr;
    const float r1 = penalty ? A.r1[h] : 0.0f, r2 = penalty ? A.r2[h] : 0.0f, sink = A.sink ? A.sink[h] : -INFINITY;
    const float slope = A.slope ? A.slope[h] : 0.0f;
    const int win = A.window > 0 ? A.window : 0x3fffffff;
    // the first key tile any row of this block sees (tiles are 64 absolute positions)
    const int j_start = attn_first_key(A, pos0 + tile * 64) / 64 * 64;
    float m_a = sink, m_b = sink, l_a = (tq == 0 && A.sink) ? 1.0f : 0.0f, l_b = l_a;
    float o[DV / 8][4];
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[nt][e] = 0.0f;
    // the next tile of keys and values is on its way (cp.async) while the current one is multiplied
    auto stage_tile = [&](int j0, int buf) {
        auto row_of = [&](int row, size_t off, int width) -> const bf16* {
            const int j = j0 + row;
            if (j > last_pos) return nullptr;
            return pool + (size_t)bt[j / A.page_size] * A.page_elems + off + ((size_t)g * A.page_size + j % A.page_size) * width;
        };
        stage_rows<DK, true>(Ks + buf * kTile, A.d, [&](int row) { return row_of(row, A.k_off, A.k_ld); });
        if (!VK) stage_rows<DV, true>(Vs + buf * kTileV, A.dv, [&](int row) { return row_of(row, A.v_off, A.v_ld); });
        cp_async_commit_group();
    };
    stage_tile(j_start, 0);
    int buf = 0;
    for (int j0 = j_start; j0 <= last_pos; j0 += 64, buf ^= 1) {
        if (j0 + 64 <= last_pos) {
            stage_tile(j0 + 64, buf ^ 1);
            cp_async_wait_group<1>();
        } else {
            cp_async_wait_group<0>();
        }
        __syncthreads();
        const bf16* Kt = Ks + buf * kTile;
        const bf16* Vt = Vs + buf * kTileV;
        if (j0 <= pos0 + tile * 64 + warp * 16 + 15 && j0 + 63 > pos0 + tile * 64 + warp * 16 - win) {      // this warp's rows see a key of the tile
            float S[8][4];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) S[nt][e] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) {
                    const bf16* p = Kt + (nt * 8 + gq) * LD + kk * 16 + tq * 2;
                    mma_bf16_16816(S[nt], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], *reinterpret_cast<const uint32_t*>(p),
                                   *reinterpret_cast<const uint32_t*>(p + 8));
                }
            float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + nt * 8 + tq * 2 + (e & 1);
                    const int i = e < 2 ? i_a : i_b;
                    const float v = (j <= i && i - j < win) ? attn_score<true>(A, S[nt][e], i - j, r1, r2, slope) : -INFINITY;
                    S[nt][e] = v;
                    if (e < 2) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            // without a sink a row of the tile's padding (beyond the sequence's rows) sees no key at all: keep its maximum finite
            const float mn_a = fmaxf(fmaxf(m_a, mx_a), -1e30f), mn_b = fmaxf(fmaxf(m_b, mx_b), -1e30f);
            const float ca = __expf(m_a - mn_a), cb = __expf(m_b - mn_b);
            m_a = mn_a; m_b = mn_b;
            l_a *= ca; l_b *= cb;
#pragma unroll
            for (int nt = 0; nt < DV / 8; ++nt) { o[nt][0] *= ca; o[nt][1] *= ca; o[nt][2] *= cb; o[nt][3] *= cb; }
            uint32_t hi[8][2], lo[8][2];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) p[e] = __expf(S[nt][e] - (e < 2 ? mn_a : mn_b));
                l_a += p[0] + p[1];
                l_b += p[2] + p[3];
                float ph[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) ph[e] = bf16_round(p[e]);
                hi[nt][0] = pack_bf16(ph[0], ph[1]); hi[nt][1] = pack_bf16(ph[2], ph[3]);
                lo[nt][0] = pack_bf16(p[0] - ph[0], p[1] - ph[1]); lo[nt][1] = pack_bf16(p[2] - ph[2], p[3] - ph[3]);
            }
#pragma unroll
            for (int k2 = 0; k2 < 4; ++k2)
#pragma unroll
                for (int nt = 0; nt < DV / 8; ++nt) {
                    uint32_t b0, b1;
                    ldmatrix_x2_trans(b0, b1, Vt + (k2 * 16 + (lane & 15)) * LDV + nt * 8);
                    mma_bf16_16816(o[nt], hi[2 * k2][0], hi[2 * k2][1], hi[2 * k2 + 1][0], hi[2 * k2 + 1][1], b0, b1);
                    mma_bf16_16816(o[nt], lo[2 * k2][0], lo[2 * k2][1], lo[2 * k2 + 1][0], lo[2 * k2 + 1][1], b0, b1);
                }
        }
        __syncthreads();
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = 1.0f / l_a, inv_b = 1.0f / l_b;
#pragma unroll
    for (int nt = 0; nt < DV / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int row = e < 2 ? row_a : row_b, c = nt * 8 + tq * 2 + (e & 1);
            if (row < n && c < A.dv) {
                const size_t t = t0 + row;
                out[t * A.out_ld + h * A.dv + c] = __float2bfloat16_rn(o[nt][e] * (e < 2 ? inv_a : inv_b) * attn_gate(A, t, h, c));
            }
        }
}

// ---------------------------------------------------------------------------------------------------------------------
// Generalized delta rule.  proj row layout: r | k | v | gate | rate (each H*d), then the decay's inner vector [rank].
struct DeltaArgs {
    const float* proj;
    int n_in, H, d, rank, n_tokens;
    float decay_coef, unit_eps, eps;
    const float *rate_bias, *decay_w2, *decay_bias, *out_norm;
    const int32_t *seq_start, *seq_pos0, *seq_slot;
    size_t slot_floats, state_off;
    int n_slots;
    int32_t* err;
};

// Per token and channel: decay w = exp(-coef * sigmoid(w2 tanh(inner) + bias)), unit key u, removal vector a * u.
__global__ void delta_prep_kernel(const DeltaArgs A, float* __restrict__ decay, float* __restrict__ ukey, float* __restrict__ aukey) {
    extern __shared__ float th[];   // tanh(inner) [rank], then per-head 1/|k|
    const int t = blockIdx.x, HD = A.H * A.d;      // blockIdx.y: a slice of blockDim.x channels
    const float* row = A.proj + (size_t)t * A.n_in;
    float* inv = th + A.rank;
    for (int r = threadIdx.x; r < A.rank; r += blockDim.x) th[r] = tanhf(row[5 * HD + r]);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int c_lo = blockIdx.y * blockDim.x, c_hi = min(HD, c_lo + blockDim.x);      // this block's channels (gridDim.y slices cover HD)
    if (c_lo >= c_hi) return;
    for (int h = c_lo / A.d + warp; h <= (c_hi - 1) / A.d; h += nw) {
        const float* k = row + HD + h * A.d;
        float ss = 0.0f;
        for (int c = lane; c < A.d; c += 32) ss += k[c] * k[c];
        ss = warp_sum(ss);
        if (lane == 0) inv[h] = 1.0f / sqrtf(ss + A.unit_eps);
    }
    __syncthreads();
    const int c = c_lo + threadIdx.x;
    if (c < c_hi) {
        float lo = A.decay_bias[c];
#pragma unroll 8
        for (int r = 0; r < A.rank; ++r) lo = fmaf(A.decay_w2[(size_t)r * HD + c], th[r], lo);
        const float u = row[HD + c] * inv[c / A.d];
        const float a = sigmoidf_(row[4 * HD + c] + A.rate_bias[c]);
        decay[(size_t)t * HD + c] = expf(-A.decay_coef * sigmoidf_(lo));
        ukey[(size_t)t * HD + c] = u;
        aukey[(size_t)t * HD + c] = a * u;
    }
}

// The recurrence.  The value columns of a head's state never mix: column j follows
//   seen = sum_i u_i S_ij;   S_ij <- w_i S_ij - (a u)_i seen + k_i v_j;   o_j = sum_i S_ij r_i
// on its own.  So a head is cut into groups of CB columns, one block per (sequence, head, group), which puts a head on
// several SMs.  L adjacent lanes share a column: lane q keeps the rows 4*(e*L + q) .. +3 (e = 0 .. R/4-1, R = DK / L,
// DK >= d key channels; channels beyond d are padded with zero keys) in registers, so that the L lanes read consecutive
// 16-byte pieces of a key-channel vector, and the two sums over key channels end with log2(L) shuffles.
// Everything a token needs (r, k, u, a u, w over the key channels; v over the block's columns) is brought into shared
// memory kDeltaChunk tokens at a time with cp.async, the next chunk while the current one is computed; inside a chunk
// the next token's vectors are read into registers before the current token is computed, so the token loop waits for
// neither global nor shared memory.  The raw o goes to global memory; delta_out_kernel finishes it.
constexpr int kDeltaChunk = 16;

__host__ __device__ constexpr int delta_lanes(int DK) { return DK >= 256 ? 16 : DK >= 64 ? 8 : 4; }
__host__ __device__ constexpr int delta_block_cols(int DK) { return DK * delta_lanes(DK) <= 128 ? DK : 128 / delta_lanes(DK); }
__host__ __device__ constexpr int delta_buf_floats(int DK) { return kDeltaChunk * (5 * DK + delta_block_cols(DK)); }

template <int VEC> __device__ __forceinline__ void cp_async_f(float* smem, const float* gmem);
template <> __device__ __forceinline__ void cp_async_f<1>(float* smem, const float* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(a), "l"(gmem));
}
template <> __device__ __forceinline__ void cp_async_f<4>(float* smem, const float* gmem) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Tokens c0 .. c0+n-1 of head h into one buffer: r | k | u | a u | w as [chunk][DK], then v of columns j0 .. j0+nc-1 as [chunk][CB].
// VEC = 4 needs d, n_in and nc to be multiples of 4 (16-byte copies).
template <int DK, int VEC>
__device__ __forceinline__ void delta_stage(const DeltaArgs& A, float* buf, int c0, int n, int h, int j0, int nc, const float* decay,
                                            const float* ukey, const float* aukey) {
    constexpr int CB = delta_block_cols(DK), PL = kDeltaChunk * DK;
    const int d = A.d, HD = A.H * d, dq = d / VEC, ncq = nc / VEC;
    for (int idx = threadIdx.x; idx < n * dq; idx += blockDim.x) {
        const int tt = idx / dq, i = (idx - tt * dq) * VEC;
        const float* prow = A.proj + (size_t)(c0 + tt) * A.n_in + h * d + i;
        const size_t vrow = (size_t)(c0 + tt) * HD + h * d + i;
        float* dst = buf + tt * DK + i;
        cp_async_f<VEC>(dst, prow);                         // r
        cp_async_f<VEC>(dst + PL, prow + HD);               // k
        cp_async_f<VEC>(dst + 2 * PL, ukey + vrow);
        cp_async_f<VEC>(dst + 3 * PL, aukey + vrow);
        cp_async_f<VEC>(dst + 4 * PL, decay + vrow);
    }
    for (int idx = threadIdx.x; idx < n * ncq; idx += blockDim.x) {
        const int tt = idx / ncq, j = (idx - tt * ncq) * VEC;
        cp_async_f<VEC>(buf + 5 * PL + tt * CB + j, A.proj + (size_t)(c0 + tt) * A.n_in + 2 * HD + h * d + j0 + j);
    }
}

// One token's vectors as a lane holds them: RV 16-byte pieces of r, k, u, a u, w and the column's v.
template <int RV>
struct DeltaToken {
    float4 r[RV], k[RV], u[RV], a[RV], w[RV];
    float v;
    __device__ __forceinline__ void load(const float4* s4, const float* s_v, int row, int row_pieces, int lanes, int plane, int cb) {
        v = s_v[row * cb];
#pragma unroll
        for (int e = 0; e < RV; ++e) {
            const float4* p = s4 + row * row_pieces + e * lanes;
            r[e] = p[0];
            k[e] = p[plane];
            u[e] = p[2 * plane];
            a[e] = p[3 * plane];
            w[e] = p[4 * plane];
        }
    }
};

template <int DK>
__global__ void __launch_bounds__(delta_block_cols(DK) * delta_lanes(DK)) delta_scan_kernel(const DeltaArgs A, const float* __restrict__ decay,
                                                                                           const float* __restrict__ ukey,
                                                                                           const float* __restrict__ aukey,
                                                                                           float* __restrict__ state_pool, float* __restrict__ o_raw) {
    constexpr int L = delta_lanes(DK), CB = delta_block_cols(DK), NS = DK / CB, RV = DK / L / 4, PL = kDeltaChunk * DK;
    constexpr int kBuf = delta_buf_floats(DK);
    static_assert(DK % (4 * L) == 0, "every lane owns whole 16-byte pieces");
    extern __shared__ __align__(16) float sh[];
    const int d = A.d, HD = A.H * d;
    const int group = blockIdx.x % NS, sh_id = blockIdx.x / NS;
    const int seq = sh_id / A.H, h = sh_id % A.H;
    const int j0 = group * CB;
    if (j0 >= d) return;                          // a group of padded columns only
    const int nc = min(CB, d - j0);
    const int col = threadIdx.x / L, q = threadIdx.x % L, j = j0 + col;
    const int t0 = A.seq_start[seq], t1 = A.seq_start[seq + 1];
    const int slot = A.seq_slot[seq];
    if (slot < 0 || slot >= A.n_slots) {
        if (threadIdx.x == 0) atomicExch(A.err, 2);
        return;
    }
    const bool vec = (d % 4 == 0) && (A.n_in % 4 == 0);
    for (int i = threadIdx.x; i < 2 * kBuf; i += blockDim.x) sh[i] = 0.0f;      // padded channels and columns stay zero for good
    __syncthreads();
    if (vec) delta_stage<DK, 4>(A, sh, t0, min(kDeltaChunk, t1 - t0), h, j0, nc, decay, ukey, aukey);
    else delta_stage<DK, 1>(A, sh, t0, min(kDeltaChunk, t1 - t0), h, j0, nc, decay, ukey, aukey);
    cp_async_commit();
    float* st = state_pool + (size_t)slot * A.slot_floats + A.state_off + (size_t)h * d * d;
    float S[RV][4];
    const bool fresh = A.seq_pos0[seq] == 0;
#pragma unroll
    for (int e = 0; e < RV; ++e)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = 4 * (e * L + q) + x;
            S[e][x] = (!fresh && i < d && j < d) ? st[(size_t)i * d + j] : 0.0f;
        }
    float po = 0.0f;                              // this lane's share of the previous token's o
    int cur = 0;
    for (int c0 = t0; c0 < t1; c0 += kDeltaChunk, cur ^= 1) {
        const int n = min(kDeltaChunk, t1 - c0);
        cp_async_wait<0>();
        __syncthreads();                          // this chunk has landed; every thread is done with the other buffer
        if (c0 + kDeltaChunk < t1) {
            const int nn = min(kDeltaChunk, t1 - c0 - kDeltaChunk);
            if (vec) delta_stage<DK, 4>(A, sh + (cur ^ 1) * kBuf, c0 + kDeltaChunk, nn, h, j0, nc, decay, ukey, aukey);
            else delta_stage<DK, 1>(A, sh + (cur ^ 1) * kBuf, c0 + kDeltaChunk, nn, h, j0, nc, decay, ukey, aukey);
            cp_async_commit();
        }
        const float* b = sh + cur * kBuf;
        const float4* s4 = reinterpret_cast<const float4*>(b) + q;      // piece e of a vector of token tt: s4[(tt*DK)/4 + e*L]
        const float* s_v = b + 5 * PL + col;
        // two register sets take turns: while one token is computed from one set, the next token's vectors land in the other
        DeltaToken<RV> ta, tb;
        ta.load(s4, s_v, 0, DK / 4, L, PL / 4, CB);
        auto step = [&](const DeltaToken<RV>& c, int tt) {
            float sa = 0.0f, sb = 0.0f;
#pragma unroll
            for (int e = 0; e < RV; ++e) {
                sa = fmaf(c.u[e].x, S[e][0], sa);
                sb = fmaf(c.u[e].y, S[e][1], sb);
                sa = fmaf(c.u[e].z, S[e][2], sa);
                sb = fmaf(c.u[e].w, S[e][3], sb);
            }
            float seen = sa + sb;
            // this token's `seen` and the previous token's o go through the shuffle stages side by side
#pragma unroll
            for (int s = 1; s < L; s <<= 1) {
                const float x = __shfl_xor_sync(0xffffffffu, seen, s), y = __shfl_xor_sync(0xffffffffu, po, s);
                seen += x;
                po += y;
            }
            if (q == 0 && j < d && c0 + tt > t0) o_raw[(size_t)(c0 + tt - 1) * HD + h * d + j] = po;
            const float ns = -seen;
            sa = 0.0f;
            sb = 0.0f;
#pragma unroll
            for (int e = 0; e < RV; ++e) {
                S[e][0] = fmaf(c.a[e].x, ns, fmaf(c.w[e].x, S[e][0], c.k[e].x * c.v));
                S[e][1] = fmaf(c.a[e].y, ns, fmaf(c.w[e].y, S[e][1], c.k[e].y * c.v));
                S[e][2] = fmaf(c.a[e].z, ns, fmaf(c.w[e].z, S[e][2], c.k[e].z * c.v));
                S[e][3] = fmaf(c.a[e].w, ns, fmaf(c.w[e].w, S[e][3], c.k[e].w * c.v));
                sa = fmaf(S[e][0], c.r[e].x, sa);
                sb = fmaf(S[e][1], c.r[e].y, sb);
                sa = fmaf(S[e][2], c.r[e].z, sa);
                sb = fmaf(S[e][3], c.r[e].w, sb);
            }
            po = sa + sb;
        };
        for (int tt = 0; tt < n; tt += 2) {
            tb.load(s4, s_v, min(tt + 1, kDeltaChunk - 1), DK / 4, L, PL / 4, CB);      // a row after the last is read and dropped
            step(ta, tt);
            if (tt + 1 < n) {
                ta.load(s4, s_v, min(tt + 2, kDeltaChunk - 1), DK / 4, L, PL / 4, CB);
                step(tb, tt + 1);
            }
        }
    }
#pragma unroll
    for (int s = 1; s < L; s <<= 1) po += __shfl_xor_sync(0xffffffffu, po, s);
    if (q == 0 && j < d && t1 > t0) o_raw[(size_t)(t1 - 1) * HD + h * d + j] = po;
#pragma unroll
    for (int e = 0; e < RV; ++e)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = 4 * (e * L + q) + x;
            if (i < d && j < d) st[(size_t)i * d + j] = S[e][x];
        }
}

// End of the recurrent mixer: each head's o divided by its root mean square, times the plain weight, times the sigmoid
// gate, written in T.  One warp per (token, head).
template <class T>
__global__ void delta_out_kernel(const DeltaArgs A, const float* __restrict__ o_raw, T* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= A.n_tokens * A.H) return;
    const int t = unit / A.H, h = unit % A.H, d = A.d, HD = A.H * d;
    const float* o = o_raw + (size_t)t * HD + h * d;
    const float* gate = A.proj + (size_t)t * A.n_in + 3 * HD + h * d;
    float ss = 0.0f;
    for (int c = lane; c < d; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)d + A.eps);
    for (int c = lane; c < d; c += 32) out[(size_t)t * HD + h * d + c] = from_f<T>(o[c] * rs * A.out_norm[h * d + c] * sigmoidf_(gate[c]));
}

// ---------------------------------------------------------------------------------------------------------------------
// Sampling: the library's integer-weight sampler, one block per row.
template <int PER>
__global__ void __launch_bounds__(kThreads) lm_sample_kernel(const float* __restrict__ logits, int n, int rows, float temp, int top_k,
                                                             float top_p, float min_p, unsigned long long seed,
                                                             const int32_t* __restrict__ seq_id, const int32_t* __restrict__ step,
                                                             int32_t* __restrict__ out) {
    extern __shared__ __align__(16) float lg[];
    __shared__ SampleScratch sc;
    for (int b = blockIdx.x; b < rows; b += gridDim.x) {
        for (int i = threadIdx.x; i < n; i += kThreads) lg[i] = logits[(size_t)b * n + i];
        __syncthreads();
        const int tok = sample_row<kThreads, PER>(lg, n, temp, top_k, top_p, min_p, seed, step ? (uint32_t)step[b] : 0u,
                                                  seq_id ? (uint32_t)seq_id[b] : (uint32_t)b, 0u, sc);
        if (threadIdx.x == 0) out[b] = tok;
        __syncthreads();
    }
}

}  // namespace lm
}  // namespace smol

#include "lm_mechanisms.cuh"
#include "lm_sigmoid_linear.cuh"

// =====================================================================================================================
// Host side
using namespace smol::lm;
using smol::bf16;

static thread_local std::string g_err;
static int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
#define CU(expr)                                                                                  \
    do {                                                                                          \
        cudaError_t e_ = (expr);                                                                  \
        if (e_ != cudaSuccess) return fail(SMOL_ERR_CUDA, std::string(#expr ": ") + cudaGetErrorString(e_)); \
    } while (0)

struct RunInfo {
    int layer;
    size_t k_off = 0, v_off = 0;   // attention: element offsets inside a page
    size_t state_off = 0;          // recurrent: float offset inside a slot
    size_t freq_off = 0;           // latent attention: float offset of the run's rotation frequencies in the table
    size_t conv_off = 0;           // state-space: float offset of the convolution's last inputs inside a slot
    int flags = 0;                 // SMOL_LM_RUN_*
};

struct SmolLm {
    SmolLmConfig cfg;
    std::vector<SmolLmLayer> layers;
    std::vector<SmolLmLayer> sides;       // sides[i]: the mixer beside layer i's (layers[i].side points here, or is null)
    std::vector<RunInfo> runs;
    std::vector<RunInfo> side_runs;       // the cache / state placement of a run's side mixer
    size_t o_conv = 0, o_head = 0;        // state-space: convolved channels [T][channels], per-head decay and step [2][T][heads]
    int max_conv = 0, max_ssd_heads = 0;
    SmolLmGlobals g{};
    size_t page_elems = 0, slot_floats = 0, esize = 2;
    int max_in = 0, max_mix = 0, max_ff = 0, max_hd = 0, max_q = 0;
    bool any_restart = false, any_own_proj = false;
    // workspace carving (byte offsets)
    size_t o_x, o_hn, o_proj, o_mix, o_y, o_z, o_act, o_dec, o_u, o_au, o_oraw, o_q, o_hw, o_err, o_part, total;
    // post-norm block: every layer result of the step; latent attention: query latent (T), full query (fp32 and T), query in
    // latent space (fp32), rotation frequencies; routed feed-forward: choices, sorted order, tile table, per-pair buffers
    size_t o_hist = 0, o_cq = 0, o_qf = 0, o_freq = 0;
    size_t o_x0 = 0, o_mix2 = 0, o_y2 = 0, o_spart = 0;
    int max_sig_cols = 0;                     // sigmoid attention: widest heads * vdim (partial sums of the tiled kernel's key ranges)    // pre-norm block: the embedding output; mixers with their own output projections: the second result
    size_t o_rlogits = 0, o_rdone = 0, o_ap = 0, o_sel_id = 0, o_sel_w = 0, o_perm = 0, o_slot_of = 0, o_seg = 0, o_tile_g = 0, o_tile_r = 0, o_ntiles = 0, o_zp = 0, o_actp = 0, o_yp = 0;
    int max_routed = 0, max_cq = 0, max_qf = 0, max_top = 0, max_experts = 0, max_pair_ff = 0;
    std::vector<float> freq_table;
    int split_len = 256, max_splits = 1, max_heads = 1, max_vdim = 1;
    char* ws = nullptr;
    void* pages = nullptr;
    float* slots = nullptr;
    int n_pages = 0, n_slots = 0;
    bool bound = false;
    bool tc_ready = false;      // the tcgen05 matrix product may be launched (attribute set, driver entry point found)
    int n_sms = 1;
    int64_t launches = 0;
    // small steps (decoding) are captured once per shape into a CUDA graph and replayed
    struct Captured { SmolLmStep key; cudaGraphExec_t exec; int64_t launches; };
    std::vector<Captured> graphs;
    cudaStream_t cap_stream = nullptr;
    ~SmolLm() {
        for (auto& g : graphs) cudaGraphExecDestroy(g.exec);
        if (cap_stream) cudaStreamDestroy(cap_stream);
    }
};

static size_t al256(size_t v) { return (v + 255) / 256 * 256; }

static int n_in_of(const SmolLmLayer& L) {
    if (L.mixer == SMOL_LM_MIX_SINK_ATTENTION) return L.heads * L.dim + L.kv_heads * L.dim + L.kv_heads * L.vdim + (L.no_gate ? 0 : L.heads * L.vdim);
    if (L.mixer == SMOL_LM_MIX_STATE_SPACE) return 2 * L.heads * L.vdim + 2 * L.bc_groups * L.n_state + L.heads;
    if (L.mixer == SMOL_LM_MIX_LATENT_ATTENTION) return L.q_rank + L.kv_rank + L.rot_dim + L.heads;
    if (L.mixer == SMOL_LM_MIX_GATED_LINEAR) return 2 * L.heads * L.dim + 2 * L.heads * L.vdim + L.rank;
    if (L.mixer == SMOL_LM_MIX_SIGMOID_ATTENTION) return L.heads * L.dim + L.kv_heads * L.dim + L.heads;
    if (L.mixer == SMOL_LM_MIX_LIGHTNING) return 2 * L.heads * L.dim + 2 * L.heads * L.vdim;
    if (L.mixer == SMOL_LM_MIX_HGRN2) return 2 * L.heads * L.dim + L.heads * L.vdim;
    return 5 * L.heads * L.dim + L.rank;
}

// columns a mixer hands to the output projection
static int mix_cols_of(const SmolLmLayer& L) { return L.mixer == SMOL_LM_MIX_GENERAL_DELTA ? L.heads * L.dim : L.heads * L.vdim; }
static bool pairable(const SmolLmLayer& L) {
    return L.mixer == SMOL_LM_MIX_SINK_ATTENTION || L.mixer == SMOL_LM_MIX_STATE_SPACE || L.mixer == SMOL_LM_MIX_SIGMOID_ATTENTION ||
           L.mixer == SMOL_LM_MIX_LIGHTNING;
}
// base^(-2i/dims) for the dims/2 rotated pairs of a latent or sigmoid attention, stretched band by band when L.rot_stretch
// is set (see the header)
static void push_frequencies(std::vector<float>& table, const SmolLmLayer& L, bool stretch) {
    const double two_pi = 6.283185307179586476925286766559;
    for (int i = 0; i < L.rot_dims / 2; ++i) {
        double f = pow((double)L.rot_base, -2.0 * i / (double)L.rot_dims);
        if (stretch && L.rot_stretch != 0.0f) {
            const double wl = two_pi / f, orig = L.rot_original;
            if (wl > orig / L.rot_low) {
                f = f / L.rot_stretch;
            } else if (wl >= orig / L.rot_high) {
                const double b = (orig / wl - L.rot_low) / ((double)L.rot_high - L.rot_low);
                f = (1.0 - b) * f / L.rot_stretch + b * f;
            }
        }
        table.push_back((float)f);
    }
}

extern "C" int smol_lm_abi_version(void) { return SMOL_LM_ABI_VERSION; }
extern "C" size_t smol_lm_struct_bytes(int which) {
    return which == 0 ? sizeof(SmolLmLayer) : which == 1 ? sizeof(SmolLmConfig) : which == 2 ? sizeof(SmolLmGlobals) : which == 3 ? sizeof(SmolLmStep) : 0;
}
extern "C" const char* smol_lm_last_error(void) { return g_err.c_str(); }

extern "C" int smol_lm_create(const SmolLmConfig* cfg, const SmolLmLayer* layers, const int32_t* run_layer, SmolLm** out) {
    if (!cfg || !layers || !run_layer || !out) return fail(SMOL_ERR_INVALID, "smol_lm_create: null argument");
    if (cfg->dtype != SMOL_LM_BF16 && cfg->dtype != SMOL_LM_F32) return fail(SMOL_ERR_INVALID, "dtype must be 0 (bf16) or 1 (f32)");
    if (cfg->vocab < 1 || cfg->width < 1 || cfg->n_layers < 1 || cfg->n_runs < 1 || cfg->page_size < 1 || cfg->max_step_tokens < 1 ||
        cfg->max_step_seqs < 1 || cfg->max_want < 1 || cfg->max_context < 1)
        return fail(SMOL_ERR_INVALID, "smol_lm_create: sizes must be positive");
    SmolLm* m = new SmolLm();
    m->cfg = *cfg;
    m->cfg.run_flags = nullptr;      // the caller's array is read below and not kept
    m->esize = cfg->dtype == SMOL_LM_F32 ? 4 : 2;
    m->layers.assign(layers, layers + cfg->n_layers);
    m->sides.resize(cfg->n_layers);
    for (int i = 0; i < cfg->n_layers; ++i)
        if (m->layers[i].side) {
            m->sides[i] = *m->layers[i].side;
            m->sides[i].side = nullptr;
            m->layers[i].side = &m->sides[i];
        }
    // places one mixer's cache or state in the pools and widens the workspace for it; returns 0 or an error code
    auto place = [&](const SmolLmLayer& L, RunInfo& r) -> int {
        if (L.heads < 1 || (L.dim < 1 && L.mixer != SMOL_LM_MIX_STATE_SPACE)) return fail(SMOL_ERR_INVALID, "a layer needs heads >= 1 and dim >= 1");
        if (L.in_bias && !pairable(L)) return fail(SMOL_ERR_UNSUPPORTED, "in_bias: softmax attention and the state-space recurrence only");
        if (L.mixer == SMOL_LM_MIX_SINK_ATTENTION) {
            if (L.kv_heads < 1 || L.heads % L.kv_heads != 0 || L.vdim < 1) return fail(SMOL_ERR_INVALID, "attention: heads must be a multiple of kv_heads");
            if (L.vdim > 32 * kAttnMaxV) return fail(SMOL_ERR_UNSUPPORTED, "attention: value size above 256");
            if (L.window < 0 || L.softcap < 0.0f) return fail(SMOL_ERR_INVALID, "attention: window and softcap must not be negative");
            r.k_off = m->page_elems;
            r.v_off = r.k_off + (size_t)L.kv_heads * cfg->page_size * L.dim;
            m->page_elems = r.v_off + (size_t)L.kv_heads * cfg->page_size * L.vdim;
            m->max_q = std::max(m->max_q, L.heads * L.dim);
            m->max_heads = std::max(m->max_heads, L.heads);
            m->max_vdim = std::max(m->max_vdim, L.vdim);
            m->max_mix = std::max(m->max_mix, L.heads * L.vdim);
        } else if (L.mixer == SMOL_LM_MIX_STATE_SPACE) {
            if (L.vdim < 1 || L.n_state < 1 || L.bc_groups < 1 || L.heads % L.bc_groups != 0 || L.conv_taps < 1 || L.norm_parts < 1 ||
                (L.heads * L.vdim) % L.norm_parts != 0)
                return fail(SMOL_ERR_INVALID, "state-space: heads must be a multiple of bc_groups, heads * vdim of norm_parts");
            if (L.n_state > 256 || L.conv_taps > kMaxTaps) return fail(SMOL_ERR_UNSUPPORTED, "state-space: state size above 256 or more than 16 taps");
            const int ch = L.heads * L.vdim + 2 * L.bc_groups * L.n_state;
            r.state_off = m->slot_floats;
            m->slot_floats += (size_t)L.heads * L.n_state * L.vdim;
            r.conv_off = m->slot_floats;
            m->slot_floats += (size_t)(L.conv_taps - 1) * ch;
            m->slot_floats = (m->slot_floats + 3) / 4 * 4;          // the next state starts on a 16-byte boundary
            m->max_hd = std::max(m->max_hd, L.heads * L.vdim);
            m->max_mix = std::max(m->max_mix, L.heads * L.vdim);
            m->max_conv = std::max(m->max_conv, ch);
            m->max_ssd_heads = std::max(m->max_ssd_heads, L.heads);
        } else if (L.mixer == SMOL_LM_MIX_GENERAL_DELTA) {
            if (L.dim > 256) return fail(SMOL_ERR_UNSUPPORTED, "recurrent mixer: key size above 256");
            if (L.rank < 1) return fail(SMOL_ERR_INVALID, "recurrent mixer: rank must be positive");
            r.state_off = m->slot_floats;
            m->slot_floats += (size_t)L.heads * L.dim * L.dim;
            m->max_hd = std::max(m->max_hd, L.heads * L.dim);
            m->max_mix = std::max(m->max_mix, L.heads * L.dim);
        } else if (L.mixer == SMOL_LM_MIX_LATENT_ATTENTION) {
            if (L.vdim < 1 || L.q_rank < 1 || L.kv_rank < 1 || L.rot_dim < 0 || L.rot_dims < 0 || L.rot_dims > L.rot_dim || L.rot_dims % 2)
                return fail(SMOL_ERR_INVALID, "latent attention: vdim, q_rank, kv_rank must be positive, rot_dims even and at most rot_dim");
            if (L.kv_rank > 32 * kAttnMaxV) return fail(SMOL_ERR_UNSUPPORTED, "latent attention: latent size above 512");
            // a cached position: the latent, then the shared rotated key part; keys and values are the same row
            r.k_off = r.v_off = m->page_elems;
            m->page_elems += (size_t)cfg->page_size * (L.kv_rank + L.rot_dim);
            r.freq_off = m->freq_table.size();
            push_frequencies(m->freq_table, L, true);
            m->max_q = std::max(m->max_q, L.heads * (L.kv_rank + L.rot_dim));
            m->max_heads = std::max(m->max_heads, L.heads);
            m->max_vdim = std::max(m->max_vdim, L.kv_rank);
            m->max_mix = std::max(m->max_mix, L.heads * std::max(L.kv_rank, L.vdim));
            m->max_hd = std::max(m->max_hd, L.heads * L.vdim);
            m->max_cq = std::max(m->max_cq, L.q_rank);
            m->max_qf = std::max(m->max_qf, L.heads * (L.dim + L.rot_dim));
        } else if (L.mixer == SMOL_LM_MIX_SIGMOID_ATTENTION) {
            if (L.kv_heads < 1 || L.heads % L.kv_heads != 0 || L.vdim != L.dim) return fail(SMOL_ERR_INVALID, "sigmoid attention: heads must be a multiple of kv_heads and vdim equal to dim");
            if (L.heads > kSigmoidMaxHeads || L.vdim > 32 * kAttnMaxV) return fail(SMOL_ERR_UNSUPPORTED, "sigmoid attention: more than 32 heads or a head size above 512");
            if (L.chunk < 0 || L.rot_dims < 0 || L.rot_dims > L.dim || L.rot_dims % 2 || !L.head_bias || !L.talk)
                return fail(SMOL_ERR_INVALID, "sigmoid attention: chunk must not be negative, rot_dims even and at most dim, head_bias and talk set");
            r.k_off = m->page_elems;
            r.v_off = r.k_off + (size_t)L.kv_heads * cfg->page_size * L.dim;
            m->page_elems = r.v_off + (size_t)L.kv_heads * cfg->page_size * L.vdim;
            r.freq_off = m->freq_table.size();
            push_frequencies(m->freq_table, L, true);
            m->max_sig_cols = std::max(m->max_sig_cols, L.heads * L.vdim);
            m->max_q = std::max(m->max_q, L.heads * L.dim);
            m->max_heads = std::max(m->max_heads, L.heads);
            m->max_vdim = std::max(m->max_vdim, L.vdim);
            m->max_mix = std::max(m->max_mix, L.heads * L.vdim);
        } else if (L.mixer == SMOL_LM_MIX_LIGHTNING || L.mixer == SMOL_LM_MIX_HGRN2) {
            if (L.dim > 256) return fail(SMOL_ERR_UNSUPPORTED, "recurrent mixer: key size above 256");
            if (L.vdim < 1 || !L.out_norm) return fail(SMOL_ERR_INVALID, "linear attention: vdim must be positive and out_norm set");
            if (L.mixer == SMOL_LM_MIX_LIGHTNING && !L.head_decay) return fail(SMOL_ERR_INVALID, "lightning attention: head_decay");
            if (L.mixer == SMOL_LM_MIX_HGRN2 && (!L.forget_lower || !L.rate_bias)) return fail(SMOL_ERR_INVALID, "HGRN2: forget_lower and rate_bias");
            r.state_off = m->slot_floats;
            m->slot_floats += (size_t)L.heads * L.dim * L.vdim;
            m->slot_floats = (m->slot_floats + 3) / 4 * 4;
            m->max_hd = std::max(m->max_hd, L.heads * std::max(L.dim, L.vdim));
            m->max_mix = std::max(m->max_mix, L.heads * L.vdim);
            if (L.mixer == SMOL_LM_MIX_LIGHTNING) {
                m->max_conv = std::max(m->max_conv, 2 * L.heads * L.dim + L.heads * L.vdim);
                m->max_ssd_heads = std::max(m->max_ssd_heads, L.heads);
            }
        } else if (L.mixer == SMOL_LM_MIX_GATED_LINEAR) {
            if (L.dim > 256) return fail(SMOL_ERR_UNSUPPORTED, "recurrent mixer: key size above 256");
            if (L.rank < 1 || L.vdim < 1 || !(L.decay_tau > 0.0f)) return fail(SMOL_ERR_INVALID, "gated linear: rank, vdim, tau must be positive");
            r.state_off = m->slot_floats;
            m->slot_floats += (size_t)L.heads * L.dim * L.vdim;
            m->max_hd = std::max(m->max_hd, L.heads * std::max(L.dim, L.vdim));
            m->max_mix = std::max(m->max_mix, L.heads * L.vdim);
        } else {
            return fail(SMOL_ERR_UNSUPPORTED, "unknown mixer kind");
        }
        return SMOL_OK;
    };
    for (int n = 0; n < cfg->n_runs; ++n) {
        const int li = run_layer[n];
        if (li < 0 || li >= cfg->n_layers) { delete m; return fail(SMOL_ERR_INVALID, "run_layer entry outside the layer array"); }
        const SmolLmLayer& L = m->layers[li];
        RunInfo r, rs;
        r.layer = rs.layer = li;
        r.flags = cfg->run_flags ? cfg->run_flags[n] : 0;
        if (r.flags & SMOL_LM_RUN_ADD_EMBED) m->any_restart = true;
        int rc = place(L, r);
        const bool prenorm = cfg->block == SMOL_LM_BLOCK_PRENORM;
        if (rc == SMOL_OK && L.side) {
            if (!pairable(L) || !pairable(*L.side)) rc = fail(SMOL_ERR_UNSUPPORTED, "mixers side by side: softmax or sigmoid attention, the state-space recurrence, lightning attention");
            else if (cfg->block == SMOL_LM_BLOCK_POSTNORM) rc = fail(SMOL_ERR_UNSUPPORTED, "mixers side by side need the sandwich or the pre-norm block");
            else if (L.proj_norm && (!prenorm || !L.side->proj_norm || !L.side->w_out)) rc = fail(SMOL_ERR_INVALID, "proj_norm: the pre-norm block, and set on both mixers with their own w_out");
            else rc = place(*L.side, rs);
            if (rc == SMOL_OK) m->max_mix = std::max(m->max_mix, mix_cols_of(L) + mix_cols_of(*L.side));
            if (rc == SMOL_OK && L.proj_norm) m->any_own_proj = true;
        }
        if (rc == SMOL_OK && prenorm) {
            if (cfg->norm_kind != SMOL_LM_NORM_RMS && cfg->norm_kind != SMOL_LM_NORM_DYT) rc = fail(SMOL_ERR_INVALID, "pre-norm block: unknown norm kind");
            else if (!L.norm1 || (L.mlp != SMOL_LM_MLP_NONE && !L.norm2)) rc = fail(SMOL_ERR_INVALID, "pre-norm block: norm weights");
            else if (cfg->norm_kind == SMOL_LM_NORM_DYT && (!L.norm1_shift || !L.norm1_alpha || (L.mlp != SMOL_LM_MLP_NONE && (!L.norm2_shift || !L.norm2_alpha))))
                rc = fail(SMOL_ERR_INVALID, "pre-norm block: the Dynamic-Tanh norms need shifts and alphas");
            else if (L.mlp == SMOL_LM_MLP_POLYNORM || L.route_input || L.out_bias || L.n_identity > 0)
                rc = fail(SMOL_ERR_UNSUPPORTED, "pre-norm block: PolyNorm feed-forwards, input-weighted routing, identity outputs and out_bias are not built");
        }
        if (rc == SMOL_OK && !prenorm && (L.shared_ff > 0 || L.proj_norm || (r.flags & SMOL_LM_RUN_ADD_EMBED) || L.mixer >= SMOL_LM_MIX_SIGMOID_ATTENTION ||
                                         (L.side && L.side->mixer >= SMOL_LM_MIX_SIGMOID_ATTENTION)))
            rc = fail(SMOL_ERR_UNSUPPORTED, "shared experts, proj_norm, restarting runs, sigmoid / lightning attention and HGRN2 need the pre-norm block");
        if (rc == SMOL_OK && L.shared_ff > 0 && (L.mlp != SMOL_LM_MLP_EXPERTS || !L.w_shared_in || !L.w_shared_out)) rc = fail(SMOL_ERR_INVALID, "shared expert: routed feed-forwards only, with both matrices");
        if (rc == SMOL_OK && cfg->block == SMOL_LM_BLOCK_POSTNORM && (L.out_bias || L.route_input))
            rc = fail(SMOL_ERR_UNSUPPORTED, "out_bias and route_input need the sandwich block");
        if (rc != SMOL_OK) { delete m; return rc; }
        if (L.mlp < SMOL_LM_MLP_NONE || L.mlp > SMOL_LM_MLP_EXPERTS) { delete m; return fail(SMOL_ERR_UNSUPPORTED, "unknown feed-forward kind"); }
        if (L.mlp == SMOL_LM_MLP_POLYNORM) m->max_ff = std::max(m->max_ff, L.ff);
        if (L.mlp == SMOL_LM_MLP_GATED || L.mlp == SMOL_LM_MLP_EXPERTS) {
            if (L.ff < 1 || L.mlp_act < SMOL_LM_ACT_GELU_TANH || L.mlp_act > SMOL_LM_ACT_RELU_SQUARED) { delete m; return fail(SMOL_ERR_INVALID, "gated feed-forward: ff and activation"); }
        }
        if (L.mlp == SMOL_LM_MLP_GATED) m->max_ff = std::max(m->max_ff, 2 * L.ff);
        if (L.mlp == SMOL_LM_MLP_EXPERTS) {
            const int E = L.n_experts + L.n_identity;
            if (L.n_experts < 0 || L.n_identity < 0 || E < 1 || E > kMaxRouted || L.top_k < 1 || L.top_k > kMaxTop || L.n_groups < 1 ||
                E % L.n_groups != 0 || L.keep_groups < 1 || L.keep_groups > L.n_groups || L.top_k > L.keep_groups * (E / L.n_groups)) {
                delete m;
                return fail(SMOL_ERR_INVALID, "routed feed-forward: experts, groups and top do not fit each other");
            }
            m->max_top = std::max(m->max_top, L.top_k);
            m->max_routed = std::max(m->max_routed, E);
            m->max_experts = std::max(m->max_experts, L.n_experts);
            m->max_pair_ff = std::max(m->max_pair_ff, L.top_k * L.ff);
            if (L.shared_ff > 0) m->max_ff = std::max(m->max_ff, (L.ff_plain ? 1 : 2) * L.shared_ff);
        }
        m->max_in = std::max(m->max_in, n_in_of(L) + (L.side ? n_in_of(*L.side) : 0));
        m->runs.push_back(r);
        m->side_runs.push_back(rs);
    }
    // pages hold 16-byte aligned rows whatever the sizes
    m->page_elems = (m->page_elems + 7) / 8 * 8;
    const size_t T = cfg->max_step_tokens, D = cfg->width, E = m->esize;
    size_t o = 0;
    auto carve = [&](size_t bytes) { size_t at = o; o += al256(bytes); return at; };
    m->o_x = carve(T * D * 4);
    m->o_hn = carve(T * D * E);
    m->o_proj = carve(T * (size_t)m->max_in * 4);
    m->o_mix = carve(T * (size_t)std::max(m->max_mix, 1) * E);
    m->o_y = carve(T * D * 4);
    m->o_z = carve(T * (size_t)std::max(m->max_ff, 1) * 4);
    m->o_act = carve(T * (size_t)std::max(m->max_ff, 1) * E);
    m->o_dec = carve(T * (size_t)std::max(m->max_hd, 1) * 4);
    m->o_u = carve(T * (size_t)std::max(m->max_hd, 1) * 4);
    m->o_au = carve(T * (size_t)std::max(m->max_hd, 1) * 4);
    m->o_oraw = carve(T * (size_t)std::max(m->max_hd, 1) * 4);
    m->o_q = carve(T * (size_t)std::max(m->max_q, 1) * E);
    m->o_hw = carve((size_t)cfg->max_want * D * E);
    m->o_err = carve(256);
    // few-token attention: key ranges of split_len positions (64 while the context stays below 16 384: a decoding row
    // then spreads over context / 64 blocks per key/value head), at most 256 of them per row; ranges are launched four at a time
    const int ctx = std::max(cfg->max_context, 1);
    m->split_len = std::max(64, ((ctx + 255) / 256 + 63) / 64 * 64);
    m->max_splits = ((ctx + m->split_len - 1) / m->split_len + 3) / 4 * 4;
    m->o_part = carve((size_t)cfg->max_step_seqs * kShortSeq * m->max_heads * m->max_splits * (m->max_vdim + 2) * 4);
    if (cfg->block == SMOL_LM_BLOCK_POSTNORM) m->o_hist = carve((size_t)(cfg->n_runs + 1) * T * D * 4);
    if (m->max_cq > 0) {
        m->o_cq = carve(T * (size_t)m->max_cq * E);
        m->o_qf = carve(T * (size_t)m->max_qf * 4);
    }
    if (!m->freq_table.empty()) m->o_freq = carve(m->freq_table.size() * 4 + 4);
    if (m->any_restart) m->o_x0 = carve(T * D * 4);
    if (m->max_sig_cols > 0 && cfg->dtype == SMOL_LM_BF16) m->o_spart = carve((size_t)kSigmoidRanges * T * m->max_sig_cols * 4);
    if (m->any_own_proj) {
        m->o_mix2 = carve(T * (size_t)std::max(m->max_mix, 1) * E);
        m->o_y2 = carve(T * D * 4);
    }
    if (m->max_conv > 0) {
        m->o_conv = carve(T * (size_t)m->max_conv * 4);
        m->o_head = carve(2 * T * (size_t)m->max_ssd_heads * 4);
    }
    if (m->max_top > 0) {
        const size_t pairs = T * (size_t)m->max_top;
        m->o_sel_id = carve(pairs * 4);
        m->o_sel_w = carve(pairs * 4);
        m->o_perm = carve(pairs * 4);
        m->o_slot_of = carve(pairs * 4);
        m->o_seg = carve(((size_t)m->max_experts + 1) * 4);
        m->o_tile_g = carve((pairs / kGroupTile + m->max_experts + 1) * 4);
        m->o_tile_r = carve((pairs / kGroupTile + m->max_experts + 1) * 4);
        m->o_ntiles = carve(4);
        m->o_zp = carve(T * (size_t)m->max_pair_ff * 2 * 4);
        m->o_actp = carve(T * (size_t)m->max_pair_ff * E);
        m->o_yp = carve(pairs * D * 4);
        m->o_ap = carve(pairs * D * E);
        m->o_rlogits = carve(T * (size_t)m->max_routed * 4);
        m->o_rdone = carve(T * 4);          // counters: zero between steps (the caller's workspace starts zeroed; the kernel resets them)
    }
    m->total = o;
    *out = m;
    return SMOL_OK;
}

extern "C" void smol_lm_destroy(SmolLm* m) { delete m; }
extern "C" size_t smol_lm_page_bytes(const SmolLm* m) { return m ? std::max<size_t>(m->page_elems, 8) * m->esize : 0; }
extern "C" size_t smol_lm_slot_bytes(const SmolLm* m) { return m ? std::max<size_t>(m->slot_floats, 4) * 4 : 0; }
extern "C" size_t smol_lm_workspace_bytes(const SmolLm* m) { return m ? m->total : 0; }
extern "C" int64_t smol_lm_launch_count(const SmolLm* m) { return m ? m->launches : 0; }
extern "C" int32_t* smol_lm_error_word(SmolLm* m) { return (m && m->bound) ? reinterpret_cast<int32_t*>(m->ws + m->o_err) : nullptr; }

template <int DK>
static cudaError_t scan_attribute() {
    cudaError_t e = cudaFuncSetAttribute(delta_scan_kernel<DK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * delta_buf_floats(DK) * sizeof(float)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gla_scan_kernel<DK, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * gla_buf_floats(DK) * sizeof(float)));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gla_scan_kernel<DK, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * gla_buf_floats(DK) * sizeof(float)));
    return e;
}
static constexpr int flash_smem_bytes(int DK, int DV, bool vk) { return 2 * 64 * ((DK + 8) + (vk ? 0 : DV + 8)) * (int)sizeof(bf16); }

template <int DK, int HPW>
static cudaError_t sigmoid_flash_attributes() {
    cudaError_t e = cudaFuncSetAttribute(sigmoid_flash_kernel<DK, HPW, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sigmoid_flash_kernel<DK, HPW, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    return e;
}

template <class T>
static cudaError_t set_kernel_attributes() {
    cudaError_t e = scan_attribute<16>();
    if (e == cudaSuccess) e = scan_attribute<32>();
    if (e == cudaSuccess) e = scan_attribute<64>();
    if (e == cudaSuccess) e = scan_attribute<128>();
    if (e == cudaSuccess) e = scan_attribute<256>();
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_split_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sigmoid_attn_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sigmoid_attn_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sigmoid_split_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSigmoidSmemMax);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sigmoid_split_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSigmoidSmemMax);
    if (e == cudaSuccess) e = sigmoid_flash_attributes<32, 1>();
    if (e == cudaSuccess) e = sigmoid_flash_attributes<64, 1>();
    if (e == cudaSuccess) e = sigmoid_flash_attributes<96, 1>();
    if (e == cudaSuccess) e = sigmoid_flash_attributes<128, 1>();
    if (e == cudaSuccess) e = sigmoid_flash_attributes<32, 2>();
    if (e == cudaSuccess) e = sigmoid_flash_attributes<64, 2>();
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_flash_kernel<128, 128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, flash_smem_bytes(128, 128, false));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_flash_kernel<192, 128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, flash_smem_bytes(192, 128, true));
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_flash_kernel<192, 192, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, flash_smem_bytes(192, 192, true));
    return e;
}

extern "C" int smol_lm_bind(SmolLm* m, const SmolLmGlobals* g, void* d_workspace, size_t workspace_bytes, void* d_pages, int32_t n_pages,
                            void* d_slots, int32_t n_slots) {
    if (!m || !g || !d_workspace || !d_pages || !d_slots) return fail(SMOL_ERR_INVALID, "smol_lm_bind: null argument");
    if (workspace_bytes < m->total) return fail(SMOL_ERR_CAPACITY, "smol_lm_bind: workspace too small");
    if (reinterpret_cast<uintptr_t>(d_workspace) % 256 || reinterpret_cast<uintptr_t>(d_pages) % 16)
        return fail(SMOL_ERR_INVALID, "smol_lm_bind: workspace must be 256-byte aligned, pages 16-byte aligned");
    if (n_pages < 1 || n_slots < 1) return fail(SMOL_ERR_INVALID, "smol_lm_bind: need at least one page and one slot");
    if (!g->embed || !g->head || !g->final_norm) return fail(SMOL_ERR_INVALID, "smol_lm_bind: missing global weights");
    CU(set_kernel_attributes<float>());
    CU(set_kernel_attributes<bf16>());
    int dev = 0;
    CU(cudaGetDevice(&dev));
    CU(cudaDeviceGetAttribute(&m->n_sms, cudaDevAttrMultiProcessorCount, dev));
    CU(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmemBytes));
    m->tc_ready = smol::tensor_map_encoder() != nullptr && m->n_sms > 0;
    m->g = *g;
    m->ws = static_cast<char*>(d_workspace);
    m->pages = d_pages;
    m->slots = static_cast<float*>(d_slots);
    m->n_pages = n_pages;
    m->n_slots = n_slots;
    if (m->cfg.block == SMOL_LM_BLOCK_POSTNORM && (size_t)m->cfg.width * 8 > 48 * 1024) {
        // the post-norm kernel keeps two fp32 copies of a row in shared memory
        if ((size_t)m->cfg.width * 8 > 200 * 1024) return fail(SMOL_ERR_UNSUPPORTED, "smol_lm_bind: width above 25600 with the post-norm block");
        CU(cudaFuncSetAttribute(post_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->cfg.width * 8));
        CU(cudaFuncSetAttribute(post_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->cfg.width * 8));
    }
    if (m->max_top > 0) CU(cudaMemset(m->ws + m->o_rdone, 0, (size_t)m->cfg.max_step_tokens * 4));      // the router's per-token counters
    if (!m->freq_table.empty())
        CU(cudaMemcpy(m->ws + m->o_freq, m->freq_table.data(), m->freq_table.size() * sizeof(float), cudaMemcpyHostToDevice));
    if (m->cfg.block == SMOL_LM_BLOCK_POSTNORM && !g->embed_norm) return fail(SMOL_ERR_INVALID, "smol_lm_bind: the post-norm block needs embed_norm");
    if (m->cfg.block == SMOL_LM_BLOCK_PRENORM && m->cfg.norm_kind == SMOL_LM_NORM_DYT && (!g->final_norm_shift || !g->final_norm_alpha))
        return fail(SMOL_ERR_INVALID, "smol_lm_bind: the Dynamic-Tanh final norm needs its shift and alpha");
    if ((size_t)m->cfg.width * 4 > 48 * 1024) {
        CU(cudaFuncSetAttribute(residual_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->cfg.width * 4));
        CU(cudaFuncSetAttribute(residual_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, m->cfg.width * 4));
    }
    m->bound = true;
    return SMOL_OK;
}

// y fp32 [M, N] = a [M, K] . w [N, K]^T
template <class T>
static cudaError_t linear(SmolLm* m, const T* a, const T* w, float* y, int M, int N, int K, cudaStream_t st);

// The general form: `io` places the operands (strides, a batch of `batch` products, or rows grouped by expert, in which
// case M is the largest number of rows and `tiles` the size of the tile table's grid; tile_rows is the table's tile height).
template <class T>
static cudaError_t linear_ex(SmolLm* m, const T* a, const T* w, float* y, int M, int N, int K, const GemmIo& io, int batch, int tiles,
                             cudaStream_t st);

template <>
cudaError_t linear_ex<float>(SmolLm* m, const float* a, const float* w, float* y, int M, int N, int K, const GemmIo& io, int batch, int tiles,
                             cudaStream_t st) {
    if (io.tile_group) {
        dim3 grid((N + 63) / 64, tiles, 1);
        gemm_f32_kernel<32, 64, 16, 2, 4><<<grid, 256, 0, st>>>(a, w, y, M, N, K, io);
    } else if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16, batch);
        gemm_f32_kernel<16, 64, 16, 1, 4><<<grid, 256, 0, st>>>(a, w, y, M, N, K, io);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
        gemm_f32_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, st>>>(a, w, y, M, N, K, io);
    }
    m->launches++;
    return cudaGetLastError();
}

template <>
cudaError_t linear<float>(SmolLm* m, const float* a, const float* w, float* y, int M, int N, int K, cudaStream_t st) {
    return linear_ex<float>(m, a, w, y, M, N, K, plain_io(K, N), 1, 0, st);
}

static bool io_vec(const void* a, const void* w, int K, const GemmIo& io) {
    const int ea = io.a_f32 ? 4 : 8;       // elements of a in 16 bytes
    return K % 8 == 0 && io.lda % ea == 0 && io.sa % ea == 0 && io.sw % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) % 16 == 0;
}

template <>
cudaError_t linear_ex<bf16>(SmolLm* m, const bf16* a, const bf16* w, float* y, int M, int N, int K, const GemmIo& io, int batch, int tiles,
                            cudaStream_t st) {
    const bool vec = io_vec(a, w, K, io);
    if (io.tile_group) {
        dim3 grid((N + 31) / 32, tiles, 1);
        gemm_bf16_kernel<1, 4, 2, 1><<<grid, 128, 0, st>>>(a, w, y, M, N, K, io, vec);       // 32 x 32
    } else if (M <= 32) {
        dim3 grid((N + 31) / 32, (M + 31) / 32, batch);
        gemm_bf16_kernel<1, 4, 2, 1><<<grid, 128, 0, st>>>(a, w, y, M, N, K, io, vec);       // 32 x 32
    } else if (M <= 256 || ((N + 63) / 64) * ((M + 127) / 128) * batch < 2 * 148) {      // 128-row tiles only when they still fill the GPU twice
        dim3 grid((N + 63) / 64, (M + 63) / 64, batch);
        gemm_bf16_kernel<2, 2, 2, 4><<<grid, 128, 0, st>>>(a, w, y, M, N, K, io, vec);       // 64 x 64
    } else {
        dim3 grid((N + 63) / 64, (M + 127) / 128, batch);
        gemm_bf16_kernel<2, 2, 4, 4><<<grid, 128, 0, st>>>(a, w, y, M, N, K, io, vec);       // 128 x 64
    }
    m->launches++;
    return cudaGetLastError();
}

template <>
cudaError_t linear<bf16>(SmolLm* m, const bf16* a, const bf16* w, float* y, int M, int N, int K, cudaStream_t st) {
    const bool aligned = K % 8 == 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) % 16 == 0;
    if (M >= kTcMinRows && N >= kTcTileN && K >= smol::umma::kBK && aligned && m->tc_ready && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
        CUtensorMap ta, tw;
        if (smol::make_tensor_map_2d(&ta, a, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)smol::umma::kM) &&
            smol::make_tensor_map_2d(&tw, w, (uint64_t)N, (uint64_t)K, (uint64_t)K, (uint32_t)kTcTileN)) {
            const int tiles = ((M + smol::umma::kM - 1) / smol::umma::kM) * ((N + kTcTileN - 1) / kTcTileN);
            gemm_tc_kernel<<<std::min(tiles, m->n_sms), kTcThreads, kTcSmemBytes, st>>>(ta, tw, y, M, N, K, plain_io(K, N));
            m->launches++;
            return cudaGetLastError();
        }
    }
    if (M <= 8 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) % 16 == 0) {
        // warps per column by N alone: a row's result must not depend on what else the step holds
        const int wpc = N >= 1184 ? 1 : N >= 592 ? 2 : 4;
        const int grid = (N * wpc + 7) / 8;
#define SMOL_GEMV(MR)                                                                                   \
        do {                                                                                            \
            if (wpc == 1) gemv_bf16_kernel<MR, 1><<<grid, 256, 0, st>>>(a, w, y, M, N, K);              \
            else if (wpc == 2) gemv_bf16_kernel<MR, 2><<<grid, 256, 0, st>>>(a, w, y, M, N, K);         \
            else gemv_bf16_kernel<MR, 4><<<grid, 256, 0, st>>>(a, w, y, M, N, K);                       \
        } while (0)
        if (M == 1) SMOL_GEMV(1);
        else if (M == 2) SMOL_GEMV(2);
        else if (M <= 4) SMOL_GEMV(4);
        else SMOL_GEMV(8);
#undef SMOL_GEMV
    } else {
        return linear_ex<bf16>(m, a, w, y, M, N, K, plain_io(K, N), 1, 0, st);
    }
    m->launches++;
    return cudaGetLastError();
}

// Grouped product on the tcgen05 tile: a [rows, K] sorted by group, w [groups * N, K], the table cut into 128-row tiles.
// Returns false if this form does not apply (then the caller takes the mma.sync form with its own table).
static bool linear_grouped_tc(SmolLm* m, const bf16* a, const bf16* w, float* y, int rows, int groups, int N, int K, const GemmIo& io,
                              cudaStream_t st) {
    const bool aligned = K % 8 == 0 && (reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w)) % 16 == 0;
    if (!(N >= kTcTileN && K >= smol::umma::kBK && aligned && m->tc_ready && reinterpret_cast<uintptr_t>(y) % 16 == 0)) return false;
    CUtensorMap ta, tw;
    if (!smol::make_tensor_map_2d(&ta, a, (uint64_t)rows, (uint64_t)K, (uint64_t)K, (uint32_t)smol::umma::kM) ||
        !smol::make_tensor_map_2d(&tw, w, (uint64_t)groups * N, (uint64_t)K, (uint64_t)K, (uint32_t)kTcTileN))
        return false;
    gemm_tc_kernel<<<m->n_sms, kTcThreads, kTcSmemBytes, st>>>(ta, tw, y, rows, N, K, io);
    m->launches++;
    return true;
}

template <int DK>
static cudaError_t launch_scan(const DeltaArgs& A, int n_seqs, const float* dec, const float* u, const float* au, float* pool, float* o_raw,
                               cudaStream_t st) {
    constexpr int threads = delta_block_cols(DK) * delta_lanes(DK), groups = DK / delta_block_cols(DK);
    delta_scan_kernel<DK><<<n_seqs * A.H * groups, threads, 2 * delta_buf_floats(DK) * sizeof(float), st>>>(A, dec, u, au, pool, o_raw);
    return cudaGetLastError();
}

template <int DK>
static cudaError_t launch_gla_scan(const GlaArgs& A, int n_seqs, const float* dec, float* pool, float* o_raw, cudaStream_t st) {
    constexpr int CB = gla_block_cols(DK), threads = CB * gla_lanes(DK);
    const int groups = (A.dv + CB - 1) / CB;
    if (A.head_decay) gla_scan_kernel<DK, true><<<n_seqs * A.H * groups, threads, 2 * gla_buf_floats(DK) * sizeof(float), st>>>(A, dec, pool, o_raw);
    else gla_scan_kernel<DK, false><<<n_seqs * A.H * groups, threads, 2 * gla_buf_floats(DK) * sizeof(float), st>>>(A, dec, pool, o_raw);
    return cudaGetLastError();
}
// the scan over key sizes up to 256: the smallest built size that holds A.d
static cudaError_t launch_gla_scan_any(const GlaArgs& A, int n_seqs, const float* dec, float* pool, float* o_raw, cudaStream_t st) {
    if (A.d <= 16) return launch_gla_scan<16>(A, n_seqs, dec, pool, o_raw, st);
    if (A.d <= 32) return launch_gla_scan<32>(A, n_seqs, dec, pool, o_raw, st);
    if (A.d <= 64) return launch_gla_scan<64>(A, n_seqs, dec, pool, o_raw, st);
    if (A.d <= 128) return launch_gla_scan<128>(A, n_seqs, dec, pool, o_raw, st);
    return launch_gla_scan<256>(A, n_seqs, dec, pool, o_raw, st);
}

// The attention kernels over the rows of a step: prompt portions on the tensor-core form (bf16, `flash`) or the
// warp-per-row form, sequences of few tokens on the split-range form.  `A` is complete except for the fields set here.
template <class T, int MAXV>
static void launch_attention(SmolLm* m, const SmolLmStep* s, AttnArgs& A, bool flash, const T* qbuf, const T* pool, T* mix, cudaStream_t st) {
    const SmolLmConfig& c = m->cfg;
    const int Tn = s->n_tokens;
    A.seq_start = s->seq_start;
    A.split_len = m->split_len;
    A.short_rows = s->n_seqs * kShortSeq;
    A.part = reinterpret_cast<float*>(m->ws + m->o_part);
    const int min_n = s->min_seq_tokens > 0 ? s->min_seq_tokens : 1;
    const int max_n = s->max_seq_tokens > 0 ? s->max_seq_tokens : Tn;
    const int max_pos = s->max_pos > 0 ? std::min(s->max_pos, c.max_context - 1) : c.max_context - 1;
    A.n_splits = std::min(m->max_splits, (max_pos / m->split_len + 4) / 4 * 4);
    if (A.window > 0) A.n_splits = std::min(A.n_splits, ((A.window - 1) / m->split_len + 2 + 3) / 4 * 4);      // ranges a window can touch
    if (max_n > kShortSeq) {
        if (flash) {
            dim3 grid((max_n + 63) / 64, s->n_seqs, A.H);
            const int hp = std::max(A.d, A.dv);
            const bf16* qb = reinterpret_cast<const bf16*>(qbuf);
            const bf16* pl = reinterpret_cast<const bf16*>(pool);
            bf16* mx = reinterpret_cast<bf16*>(mix);
#define SMOL_FLASH(DK, DV, VK) attn_flash_kernel<DK, DV, VK><<<grid, 128, flash_smem_bytes(DK, DV, VK), st>>>(A, qb, pl, mx)
            if (A.v_in_k) {
                if (A.d <= 64) SMOL_FLASH(64, 64, true);
                else if (A.d <= 128) SMOL_FLASH(128, 128, true);
                else if (A.dv <= 128) SMOL_FLASH(192, 128, true);
                else SMOL_FLASH(192, 192, true);
            } else if (hp <= 32) SMOL_FLASH(32, 32, false);
            else if (hp <= 64) SMOL_FLASH(64, 64, false);
            else SMOL_FLASH(128, 128, false);
#undef SMOL_FLASH
        } else {
            // every row, also those of short sequences
            const int au = Tn * A.H;
            attn_kernel<T, MAXV><<<(au + kAttnWarps - 1) / kAttnWarps, kAttnWarps * 32, kAttnWarps * A.d * sizeof(float), st>>>(A, qbuf, pool, mix);
        }
        m->launches += 1;
    }
    if (min_n <= kShortSeq && (flash || max_n <= kShortSeq)) {
        const int Gq = A.H / A.G, nwarp = std::min(Gq, 8), groups = (Gq + nwarp - 1) / nwarp;
        const int pad = 16 / (int)sizeof(T);
        const size_t smem = ((size_t)nwarp * (A.d + 32) * 4 + 15) / 16 * 16 + (size_t)32 * (A.d + pad + (A.v_in_k ? 0 : A.dv + pad)) * sizeof(T);
        dim3 grid(A.short_rows, A.G * groups, A.n_splits);
        attn_split_kernel<T, MAXV><<<grid, nwarp * 32, smem, st>>>(A, qbuf, pool);
        attn_merge_kernel<T, MAXV><<<(A.short_rows * A.H + 3) / 4, 128, 0, st>>>(A, mix);
        m->launches += 2;
    }
}

// The tiled sigmoid attention over the sequences that bring more than kShortSeq tokens.  Returns false where this form does
// not apply (fp32 engine, sizes it is not built for, unaligned cached rows, more shared memory than an SM has): the caller
// then runs the warp-per-head kernel over every row.
static size_t sigmoid_flash_smem(int H, int G, int DK, int KT) {
    return (size_t)2 * G * KT * (DK + 8) * sizeof(bf16) + ((size_t)H * 16 * (KT + 8) + (size_t)H * H) * sizeof(float);
}
template <int DK, int HPW>
static bool launch_sigmoid_flash_sized(const SigmoidArgs& S, dim3 grid, int threads, const bf16* qbuf, const bf16* pool, bf16* out, cudaStream_t st) {
    const AttnArgs& A = S.a;
    if (sigmoid_flash_smem(A.H, A.G, DK, 64) <= (size_t)kSigmoidSmemMax) {
        sigmoid_flash_kernel<DK, HPW, 64><<<grid, threads, sigmoid_flash_smem(A.H, A.G, DK, 64), st>>>(S, qbuf, pool, out);
        return true;
    }
    if (sigmoid_flash_smem(A.H, A.G, DK, 32) <= (size_t)kSigmoidSmemMax) {
        sigmoid_flash_kernel<DK, HPW, 32><<<grid, threads, sigmoid_flash_smem(A.H, A.G, DK, 32), st>>>(S, qbuf, pool, out);
        return true;
    }
    return false;
}
static bool launch_sigmoid_flash(SmolLm* m, const SmolLmStep* s, SigmoidArgs& S, int max_n, const bf16* qbuf, const bf16* pool, bf16* out,
                                 bool is_bf16, cudaStream_t st) {
    const AttnArgs& A = S.a;
    if (!is_bf16 || A.d % 8 != 0 || A.d > 128 || A.k_off % 8 != 0 || A.v_off % 8 != 0) return false;
    // Key ranges: a quarter of the positions a row tile can see (at least 256, whole 64-key tiles), more only where that
    // would cut a tile into more than kSigmoidRanges ranges.  The ranges depend on the mask and the pool's size alone.
    const int span = S.chunk > 0 ? std::min(S.chunk + 15, m->cfg.max_context) : m->cfg.max_context;
    auto ranges_of = [&](int len) { return S.chunk > 0 ? (span + len - 1) / len + 1 : (span + len - 1) / len; };
    int len = std::max(256, ((span + 3) / 4 + 63) / 64 * 64);
    while (ranges_of(len) > kSigmoidRanges) len += 64;
    S.range_len = len;
    S.n_ranges = ranges_of(len);
    if (span <= 512) {                       // few keys per row: one range, the result written directly
        S.range_len = 1 << 30;
        S.n_ranges = 1;
    }
    S.partial = reinterpret_cast<float*>(m->ws + m->o_spart);
    const dim3 grid((max_n + 15) / 16, s->n_seqs, S.n_ranges);
    bool done;
    if (A.H <= 16) {
        const int threads = A.H * 32;
        if (A.d <= 32) done = launch_sigmoid_flash_sized<32, 1>(S, grid, threads, qbuf, pool, out, st);
        else if (A.d <= 64) done = launch_sigmoid_flash_sized<64, 1>(S, grid, threads, qbuf, pool, out, st);
        else if (A.d <= 96) done = launch_sigmoid_flash_sized<96, 1>(S, grid, threads, qbuf, pool, out, st);
        else done = launch_sigmoid_flash_sized<128, 1>(S, grid, threads, qbuf, pool, out, st);
    } else {
        const int threads = (A.H + 1) / 2 * 32;
        if (A.d <= 32) done = launch_sigmoid_flash_sized<32, 2>(S, grid, threads, qbuf, pool, out, st);
        else if (A.d <= 64) done = launch_sigmoid_flash_sized<64, 2>(S, grid, threads, qbuf, pool, out, st);
        else done = false;
    }
    if (done && S.n_ranges > 1) {
        sigmoid_merge_kernel<<<A.n_tokens, 128, 0, st>>>(S, out);
        m->launches += 1;
    }
    if (done) m->launches += 1;
    return done;
}

template <class T>
static int step_impl(SmolLm* m, const SmolLmStep* s, cudaStream_t st) {
    const SmolLmConfig& c = m->cfg;
    const int Tn = s->n_tokens, D = c.width;
    float* x = reinterpret_cast<float*>(m->ws + m->o_x);
    T* hn = reinterpret_cast<T*>(m->ws + m->o_hn);
    float* proj = reinterpret_cast<float*>(m->ws + m->o_proj);
    T* mix = reinterpret_cast<T*>(m->ws + m->o_mix);
    float* y = reinterpret_cast<float*>(m->ws + m->o_y);
    float* z = reinterpret_cast<float*>(m->ws + m->o_z);
    T* act = reinterpret_cast<T*>(m->ws + m->o_act);
    float* dec = reinterpret_cast<float*>(m->ws + m->o_dec);
    float* uk = reinterpret_cast<float*>(m->ws + m->o_u);
    float* auk = reinterpret_cast<float*>(m->ws + m->o_au);
    float* oraw = reinterpret_cast<float*>(m->ws + m->o_oraw);
    T* qbuf = reinterpret_cast<T*>(m->ws + m->o_q);
    T* hw = reinterpret_cast<T*>(m->ws + m->o_hw);
    int32_t* err = reinterpret_cast<int32_t*>(m->ws + m->o_err);
    float* hist = reinterpret_cast<float*>(m->ws + m->o_hist);
    T* pool = static_cast<T*>(m->pages);
    const int nthr = D >= 1024 ? 256 : 128;
    const bool postnorm = c.block == SMOL_LM_BLOCK_POSTNORM, prenorm = c.block == SMOL_LM_BLOCK_PRENORM;
    float* x0 = m->any_restart ? reinterpret_cast<float*>(m->ws + m->o_x0) : nullptr;
    T* mix2 = reinterpret_cast<T*>(m->ws + m->o_mix2);
    float* y2 = reinterpret_cast<float*>(m->ws + m->o_y2);
    auto norm_of = [&](const float* w, const float* shift, const float* alpha) { return NormSpec{c.norm_kind, w, shift, alpha, c.norm_eps}; };
    const NormSpec no_norm{c.norm_kind, nullptr, nullptr, nullptr, c.norm_eps};
    const size_t hist_stride = (size_t)Tn * D;
    constexpr bool kIsF32 = sizeof(T) == 4;
    const float woff = c.norm_plain ? 0.0f : 1.0f;
    float* conv = reinterpret_cast<float*>(m->ws + m->o_conv);
    float* head = reinterpret_cast<float*>(m->ws + m->o_head);
    auto cast_grid = [](size_t n) { return (int)std::min<size_t>((n + 255) / 256, 148 * 8); };

    if (postnorm) {
        embed_gain_norm_kernel<T><<<Tn, nthr, 0, st>>>(s->tokens, static_cast<const T*>(m->g.embed), D, c.vocab, m->g.embed_norm, c.norm_eps, x, hist, hn);
    } else if (prenorm) {
        const SmolLmLayer& L0 = m->layers[m->runs[0].layer];
        embed_prenorm_kernel<T><<<Tn, nthr, 0, st>>>(s->tokens, static_cast<const T*>(m->g.embed), c.embed_scale, D, c.vocab,
                                                     norm_of(L0.norm1, L0.norm1_shift, L0.norm1_alpha), x, x0, hn);
    } else {
        embed_norm_kernel<T><<<Tn, nthr, 0, st>>>(s->tokens, static_cast<const T*>(m->g.embed), c.embed_scale, D, c.vocab,
                                                  m->layers[m->runs[0].layer].norm1, c.norm_eps, x, hn, woff);
    }
    m->launches++;
    for (size_t n = 0; n < m->runs.size(); ++n) {
        const RunInfo& R = m->runs[n];
        const SmolLmLayer& L = m->layers[R.layer];
        const int n_in_main = n_in_of(L), n_in = n_in_main + (L.side ? n_in_of(*L.side) : 0);
        CU(linear<T>(m, hn, static_cast<const T*>(L.w_in), proj, Tn, n_in, D, st));
        const int mix_ld = mix_cols_of(L) + (L.side ? mix_cols_of(*L.side) : 0);      // row stride of the mixers' shared result
        int mix_cols;
        int out_ld_now = mix_ld;        // row stride of the buffer the current mixer writes
        const T* mix_in = mix;          // what the output projection reads
        // Softmax attention over keys and values in the paged pool.  pj / bias: this mixer's rows of the fused projection.
        auto attention = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj, const float* bias, T* mix_at) -> int {
            AttnArgs A;
            A.proj = pj; A.n_in = n_in; A.bias = bias;
            A.tok_seq = s->tok_seq; A.tok_pos = s->tok_pos; A.block_table = s->block_table;
            A.max_pages = s->max_pages; A.page_size = c.page_size; A.n_pages = m->n_pages;
            A.page_elems = m->page_elems; A.k_off = Ri.k_off; A.v_off = Ri.v_off;
            A.H = M.heads; A.scale = M.score_scale; A.eps = c.norm_eps;
            A.n_tokens = Tn; A.err = err;
            A.G = M.kv_heads; A.d = M.dim; A.dv = M.vdim;
            A.k_ld = M.dim; A.v_ld = M.vdim; A.v_in_k = 0;
            A.gate_off = (size_t)M.heads * M.dim + (size_t)M.kv_heads * (M.dim + M.vdim); A.gate_ld = M.vdim; A.gate_step = 1;
            A.has_gate = M.no_gate ? 0 : 1;
            A.q_norm = M.q_norm; A.k_norm = M.k_norm; A.r1 = M.dist_r1; A.r2 = M.dist_r2; A.sink = M.sink;
            A.slope = M.dist_slope; A.window = M.window; A.softcap = M.softcap; A.two_over_cap = M.softcap > 0.0f ? 2.0f / M.softcap : 0.0f;
            A.out_ld = out_ld_now; A.out_scale = M.mix_scale;
            if (M.norm_whole) {
                attn_prep_whole_kernel<T><<<Tn, Tn > 64 ? 128 : 256, 0, st>>>(A, qbuf, pool);      // few tokens: more loads in flight per token
            } else {
                const int units = Tn * (M.heads + 2 * M.kv_heads);
                attn_prep_kernel<T><<<(units + 3) / 4, 128, 0, st>>>(A, qbuf, pool);
            }
            m->launches += 1;
            const bool flash = sizeof(T) == 2 && std::max(M.dim, M.vdim) <= 128;
            if (M.vdim <= 256) launch_attention<T, 8>(m, s, A, flash, qbuf, pool, mix_at, st);
            else launch_attention<T, 16>(m, s, A, flash, qbuf, pool, mix_at, st);
            return SMOL_OK;
        };
        // State-space recurrence: convolution and per-head step / decay, the scan over the slot's state, then skip, gate and the
        // grouped norm (whose kernel also leaves the slot's new convolution inputs).
        auto state_space = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj, const float* bias, T* mix_at) -> int {
            const int inner = M.heads * M.vdim, gn = M.bc_groups * M.n_state, ch = inner + 2 * gn;
            SsdArgs P;
            P.proj = pj; P.bias = bias; P.n_in = n_in; P.H = M.heads; P.dv = M.vdim; P.N = M.n_state; P.G = M.bc_groups;
            P.taps = M.conv_taps; P.parts = M.norm_parts; P.n_tokens = Tn; P.n_seqs = s->n_seqs; P.eps = c.norm_eps;
            P.conv_w = M.conv_w; P.conv_b = M.conv_b; P.dt_bias = M.dt_bias; P.a_log = M.a_log; P.skip = M.skip; P.out_norm = M.out_norm;
            P.seq_start = s->seq_start; P.seq_pos0 = s->seq_pos0; P.seq_slot = s->seq_slot; P.tok_seq = s->tok_seq;
            P.slot_floats = m->slot_floats; P.conv_off = Ri.conv_off; P.n_slots = m->n_slots; P.err = err;
            P.out_ld = out_ld_now; P.out_scale = M.mix_scale;
            const dim3 cgrid(Tn, (ch + 127) / 128);
            ssd_conv_kernel<<<cgrid, 128, 0, st>>>(P, m->slots, conv, head);
            GlaArgs A;
            A.proj = pj; A.n_in = n_in; A.H = M.heads; A.d = M.n_state; A.dv = M.vdim; A.rank = 0; A.n_tokens = Tn;
            A.q_scale = 1.0f; A.tau = 1.0f; A.eps = c.norm_eps;
            A.decay_w2 = A.decay_bias = A.out_norm = nullptr;
            A.seq_start = s->seq_start; A.seq_pos0 = s->seq_pos0; A.seq_slot = s->seq_slot;
            A.slot_floats = m->slot_floats; A.state_off = Ri.state_off; A.n_slots = m->n_slots; A.err = err;
            A.q_src = conv + inner + gn; A.k_src = conv + inner; A.v_src = conv;
            A.q_ld = A.k_ld = A.v_ld = ch;
            A.qk_share = M.heads / M.bc_groups;
            A.head_decay = head; A.head_step = head + (size_t)Tn * M.heads;
            A.out_ld = out_ld_now; A.out_scale = 1.0f;
            CU(launch_gla_scan_any(A, s->n_seqs, nullptr, m->slots, oraw, st));
            ssd_out_kernel<T><<<dim3(Tn, M.norm_parts), 256, 0, st>>>(P, oraw, conv, mix_at, m->slots);
            m->launches += 3;
            return SMOL_OK;
        };
        // Mixers side by side that own their output projections keep their results apart: row stride = own columns.
        const bool own_proj = L.side && L.proj_norm;
        // Sigmoid attention over keys and values in the paged pool.
        auto sigmoid_attention = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj, const float* bias, T* mix_at, int ld) -> int {
            SigmoidArgs S;
            AttnArgs& A = S.a;
            A.proj = pj; A.n_in = n_in; A.bias = bias;
            A.tok_seq = s->tok_seq; A.tok_pos = s->tok_pos; A.block_table = s->block_table;
            A.max_pages = s->max_pages; A.page_size = c.page_size; A.n_pages = m->n_pages;
            A.page_elems = m->page_elems; A.k_off = Ri.k_off; A.v_off = Ri.v_off;
            A.H = M.heads; A.G = M.kv_heads; A.d = M.dim; A.dv = M.vdim; A.scale = M.score_scale; A.eps = c.norm_eps;
            A.n_tokens = Tn; A.err = err; A.seq_start = s->seq_start;
            A.k_ld = M.dim; A.v_ld = M.vdim; A.v_in_k = 0;
            A.gate_off = (size_t)(M.heads + M.kv_heads) * M.dim; A.gate_ld = 1; A.gate_step = 0; A.has_gate = 1;
            A.q_norm = A.k_norm = A.r1 = A.r2 = A.sink = A.slope = nullptr;
            A.window = 0; A.softcap = A.two_over_cap = 0.0f;
            A.split_len = A.n_splits = A.short_rows = 0; A.part = nullptr;
            A.out_ld = ld; A.out_scale = 1.0f;
            S.chunk = M.chunk; S.rot_pairs = M.rot_dims / 2; S.head_bias = M.head_bias; S.talk = M.talk; S.only = 0;
            S.range_len = 1 << 30; S.n_ranges = 1; S.partial = nullptr;
            S.freq = reinterpret_cast<const float*>(m->ws + m->o_freq) + Ri.freq_off;
            const int units = Tn * (M.heads + M.kv_heads);
            sigmoid_prep_kernel<T><<<(units + 3) / 4, 128, 0, st>>>(S, qbuf, pool);
            m->launches += 1;
            const int min_n = s->min_seq_tokens > 0 ? s->min_seq_tokens : 1;
            const int max_n = s->max_seq_tokens > 0 ? s->max_seq_tokens : Tn;
            // sequences that bring more than a few tokens take the tiled tensor-core form (bf16), the others a warp per head
            const bool tiled = max_n > kShortSeq && launch_sigmoid_flash(m, s, S, max_n, reinterpret_cast<const bf16*>(qbuf), reinterpret_cast<const bf16*>(pool),
                                                                         reinterpret_cast<bf16*>(mix_at), sizeof(T) == 2, st);
            // sequences of few tokens (decoding): key ranges over separate blocks, merged afterwards
            const size_t split_smem = sigmoid_split_smem<T>(M.heads, M.kv_heads, M.dim, M.vdim);
            const bool split = min_n <= kShortSeq && split_smem <= (size_t)kSigmoidSmemMax;
            if (split) {
                const int max_pos = s->max_pos > 0 ? std::min(s->max_pos, c.max_context - 1) : c.max_context - 1;
                A.split_len = m->split_len;
                A.short_rows = s->n_seqs * kShortSeq;
                A.part = reinterpret_cast<float*>(m->ws + m->o_part);
                A.n_splits = std::min(m->max_splits, (max_pos / m->split_len + 4) / 4 * 4);
                if (M.chunk > 0) A.n_splits = std::min(A.n_splits, ((M.chunk - 1) / m->split_len + 2 + 3) / 4 * 4);      // ranges a chunk can touch
                const dim3 grid(A.short_rows, A.n_splits);
                if (M.vdim <= 256) sigmoid_split_kernel<T, 8><<<grid, M.heads * 32, split_smem, st>>>(S, qbuf, pool);
                else sigmoid_split_kernel<T, 16><<<grid, M.heads * 32, split_smem, st>>>(S, qbuf, pool);
                sigmoid_short_merge_kernel<T><<<A.short_rows, 128, 0, st>>>(S, mix_at);
                m->launches += 2;
            }
            const bool long_left = max_n > kShortSeq && !tiled, short_left = min_n <= kShortSeq && !split;
            if (long_left || short_left) {
                // the warp-per-head form: every row, or only the rows the other two forms left
                S.only = (long_left && short_left) ? 0 : long_left ? 1 : 2;
                const size_t smem = ((size_t)M.heads * (M.dim + 32) + (size_t)M.heads * M.heads) * sizeof(float);
                if (M.vdim <= 256) sigmoid_attn_kernel<T, 8><<<Tn, M.heads * 32, smem, st>>>(S, qbuf, pool, mix_at);
                else sigmoid_attn_kernel<T, 16><<<Tn, M.heads * 32, smem, st>>>(S, qbuf, pool, mix_at);
                m->launches += 1;
            }
            return SMOL_OK;
        };
        // The scan's arguments for a linear attention with state [dim, vdim] per head in the slot.
        auto scan_args = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj) {
            GlaArgs A;
            A.proj = pj; A.n_in = n_in; A.H = M.heads; A.d = M.dim; A.dv = M.vdim; A.rank = 0; A.n_tokens = Tn;
            A.q_scale = 1.0f; A.tau = 1.0f; A.eps = c.norm_eps;
            A.decay_w2 = A.decay_bias = A.out_norm = nullptr;
            A.seq_start = s->seq_start; A.seq_pos0 = s->seq_pos0; A.seq_slot = s->seq_slot;
            A.slot_floats = m->slot_floats; A.state_off = Ri.state_off; A.n_slots = m->n_slots; A.err = err;
            A.qk_share = 1; A.head_decay = A.head_step = nullptr;
            A.out_ld = M.heads * M.vdim; A.out_scale = 1.0f;
            return A;
        };
        // Lightning attention: silu on q, k, v; the scan in its one-decay-per-head form; norm over all heads, sigmoid gate.
        auto lightning = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj, T* mix_at, int ld) -> int {
            const int hd = M.heads * M.dim, hv = M.heads * M.vdim, na = 2 * hd + hv;
            LinPrepArgs P{pj, n_in, M.heads, M.dim, M.vdim, Tn, M.head_decay, nullptr, nullptr};
            lightning_prep_kernel<<<dim3(Tn, (na + 1023) / 1024), 256, 0, st>>>(P, conv, head);
            GlaArgs A = scan_args(M, Ri, pj);
            A.q_src = conv; A.k_src = conv + hd; A.v_src = conv + 2 * hd;
            A.q_ld = A.k_ld = A.v_ld = na;
            A.head_decay = head; A.head_step = head + (size_t)Tn * M.heads;
            CU(launch_gla_scan_any(A, s->n_seqs, nullptr, m->slots, oraw, st));
            LinOutArgs O{pj, n_in, hv, hv, hv, 1, ld, (size_t)2 * hd + hv, c.norm_eps, 1.0f, M.out_norm};
            lin_attn_out_kernel<T><<<dim3(Tn, 1), 256, 0, st>>>(O, oraw, mix_at);
            m->launches += 3;
            return SMOL_OK;
        };
        auto run_mixer = [&](const SmolLmLayer& M, const RunInfo& Ri, const float* pj, const float* bias, T* mix_at, int ld) -> int {
            out_ld_now = ld;
            if (M.mixer == SMOL_LM_MIX_SINK_ATTENTION) return attention(M, Ri, pj, bias, mix_at);
            if (M.mixer == SMOL_LM_MIX_STATE_SPACE) return state_space(M, Ri, pj, bias, mix_at);
            if (M.mixer == SMOL_LM_MIX_SIGMOID_ATTENTION) return sigmoid_attention(M, Ri, pj, bias, mix_at, ld);
            return lightning(M, Ri, pj, mix_at, ld);
        };
        if (pairable(L)) {
            int rc = run_mixer(L, R, proj, L.in_bias, mix, own_proj ? mix_cols_of(L) : mix_ld);
            if (rc == SMOL_OK && L.side) {
                const SmolLmLayer& S = *L.side;
                const float* sb = L.in_bias ? L.in_bias + n_in_main : nullptr;
                rc = run_mixer(S, m->side_runs[n], proj + n_in_main, sb, own_proj ? mix2 : mix + mix_cols_of(L), own_proj ? mix_cols_of(S) : mix_ld);
            }
            if (rc != SMOL_OK) return rc;
            mix_cols = own_proj ? mix_cols_of(L) : mix_ld;
        } else if (L.mixer == SMOL_LM_MIX_HGRN2) {
            // q = silu(.), decay = the bounded forget gate, key = 1 - decay; norm per head, no gate
            const int hd = L.heads * L.dim, hv = L.heads * L.vdim;
            LinPrepArgs P{proj, n_in, L.heads, L.dim, L.vdim, Tn, nullptr, L.rate_bias, L.forget_lower};
            hgrn2_prep_kernel<<<dim3(Tn, (hd + 1023) / 1024), 256, 0, st>>>(P, uk, auk, dec);
            GlaArgs A = scan_args(L, R, proj);
            A.q_src = uk; A.k_src = auk; A.v_src = proj + 2 * hd;
            A.q_ld = A.k_ld = hd; A.v_ld = n_in;
            CU(launch_gla_scan_any(A, s->n_seqs, dec, m->slots, oraw, st));
            LinOutArgs O{proj, n_in, hv, L.vdim, L.vdim, 0, hv, 0, c.norm_eps, 1.0f, L.out_norm};
            lin_attn_out_kernel<T><<<dim3(Tn, L.heads), 128, 0, st>>>(O, oraw, mix);
            m->launches += 3;
            mix_cols = hv;
        } else if (L.mixer == SMOL_LM_MIX_LATENT_ATTENTION) {
            AttnArgs A;
            A.proj = proj; A.n_in = n_in; A.bias = nullptr;
            A.tok_seq = s->tok_seq; A.tok_pos = s->tok_pos; A.block_table = s->block_table;
            A.max_pages = s->max_pages; A.page_size = c.page_size; A.n_pages = m->n_pages;
            A.page_elems = m->page_elems; A.k_off = R.k_off; A.v_off = R.v_off;
            A.H = L.heads; A.scale = L.score_scale; A.eps = c.norm_eps;
            A.n_tokens = Tn; A.err = err;
            A.slope = nullptr; A.window = 0; A.softcap = A.two_over_cap = 0.0f; A.has_gate = 1; A.out_scale = 1.0f; A.out_ld = L.heads * L.kv_rank;
            {
                const int dk = L.kv_rank + L.rot_dim, qw = L.dim + L.rot_dim;
                T* cq = reinterpret_cast<T*>(m->ws + m->o_cq);
                float* qf = reinterpret_cast<float*>(m->ws + m->o_qf);
                LatentArgs P;
                P.proj = proj; P.n_in = n_in; P.q_rank = L.q_rank; P.kv_rank = L.kv_rank; P.rot = L.rot_dim; P.rot_pairs = L.rot_dims / 2; P.H = L.heads; P.d = L.dim;
                P.eps = c.norm_eps; P.q_lat_norm = L.q_lat_norm; P.kv_lat_norm = L.kv_lat_norm;
                P.freq = reinterpret_cast<const float*>(m->ws + m->o_freq) + R.freq_off;
                P.tok_seq = s->tok_seq; P.tok_pos = s->tok_pos; P.block_table = s->block_table;
                P.max_pages = s->max_pages; P.page_size = c.page_size; P.n_pages = m->n_pages; P.n_tokens = Tn;
                P.page_elems = m->page_elems; P.k_off = R.k_off; P.err = err;
                latent_prep_kernel<T><<<Tn, 128, 0, st>>>(P, cq, pool);
                CU(linear<T>(m, cq, static_cast<const T*>(L.w_q_up), qf, Tn, L.heads * qw, L.q_rank, st));
                // per head: the unrotated query [Tn, dim] times the transposed key expansion [kv_rank, dim]^T, written where
                // the attention reads its queries (bf16 engine: read from the fp32 q, written in bf16)
                GemmIo io = plain_io(L.dim, L.kv_rank);
                io.lda = L.heads * qw; io.ldy = L.heads * dk;
                io.sa = qw; io.sw = (long long)L.kv_rank * L.dim; io.sy = dk;
                io.a_f32 = io.y_bf16 = kIsF32 ? 0 : 1;
                CU(linear_ex<T>(m, reinterpret_cast<const T*>(qf), static_cast<const T*>(L.w_k_up_t), reinterpret_cast<float*>(qbuf), Tn, L.kv_rank,
                                L.dim, io, L.heads, 0, st));
                latent_query_kernel<T><<<(Tn * L.heads + 3) / 4, 128, 0, st>>>(P, qf, qbuf);
                m->launches += 2;
                A.G = 1; A.d = dk; A.dv = L.kv_rank;
                A.k_ld = dk; A.v_ld = dk; A.v_in_k = 1;
                A.gate_off = (size_t)L.q_rank + dk; A.gate_ld = 1; A.gate_step = 0;
                A.q_norm = A.k_norm = A.r1 = A.r2 = A.sink = nullptr;
                const bool flash = sizeof(T) == 2 && dk <= 192;          // larger latents take the warp-per-row form for prompt portions
                if (L.kv_rank <= 256) launch_attention<T, 8>(m, s, A, flash, qbuf, pool, mix, st);
                else launch_attention<T, 16>(m, s, A, flash, qbuf, pool, mix, st);
                // per head: the attended latent [Tn, kv_rank] times the value expansion [vdim, kv_rank]^T
                GemmIo iv = plain_io(L.kv_rank, L.vdim);
                iv.lda = L.heads * L.kv_rank; iv.ldy = L.heads * L.vdim;
                iv.sa = L.kv_rank; iv.sw = (long long)L.vdim * L.kv_rank; iv.sy = L.vdim;
                iv.y_bf16 = kIsF32 ? 0 : 1;
                T* expanded = reinterpret_cast<T*>(oraw);          // [Tn, heads * vdim] in T
                CU(linear_ex<T>(m, mix, static_cast<const T*>(L.w_v_up), reinterpret_cast<float*>(expanded), Tn, L.vdim, L.kv_rank, iv, L.heads, 0, st));
                mix_cols = L.heads * L.vdim;
                mix_in = expanded;
            }
        } else if (L.mixer == SMOL_LM_MIX_GATED_LINEAR) {
            GlaArgs A;
            A.proj = proj; A.n_in = n_in; A.H = L.heads; A.d = L.dim; A.dv = L.vdim; A.rank = L.rank; A.n_tokens = Tn;
            A.q_scale = L.score_scale; A.tau = L.decay_tau; A.eps = c.norm_eps;
            A.decay_w2 = L.decay_w2; A.decay_bias = L.decay_bias; A.out_norm = L.out_norm;
            A.seq_start = s->seq_start; A.seq_pos0 = s->seq_pos0; A.seq_slot = s->seq_slot;
            A.slot_floats = m->slot_floats; A.state_off = R.state_off; A.n_slots = m->n_slots; A.err = err;
            gla_sources_from_proj(A);
            gla_prep_kernel<<<dim3(Tn, (L.heads * L.dim + 127) / 128), 128, L.rank * sizeof(float), st>>>(A, dec);
            CU(launch_gla_scan_any(A, s->n_seqs, dec, m->slots, oraw, st));
            gla_out_kernel<T><<<(Tn * L.heads + 3) / 4, 128, 0, st>>>(A, oraw, mix);
            m->launches += 3;
            mix_cols = L.heads * L.vdim;
        } else {
            DeltaArgs A;
            A.proj = proj; A.n_in = n_in; A.H = L.heads; A.d = L.dim; A.rank = L.rank; A.n_tokens = Tn;
            A.decay_coef = L.decay_coef; A.unit_eps = L.unit_eps; A.eps = c.norm_eps;
            A.rate_bias = L.rate_bias; A.decay_w2 = L.decay_w2; A.decay_bias = L.decay_bias; A.out_norm = L.out_norm;
            A.seq_start = s->seq_start; A.seq_pos0 = s->seq_pos0; A.seq_slot = s->seq_slot;
            A.slot_floats = m->slot_floats; A.state_off = R.state_off; A.n_slots = m->n_slots; A.err = err;
            delta_prep_kernel<<<dim3(Tn, (L.heads * L.dim + 127) / 128), 128, (L.rank + L.heads) * sizeof(float), st>>>(A, dec, uk, auk);
            cudaError_t e;
            if (L.dim <= 16) e = launch_scan<16>(A, s->n_seqs, dec, uk, auk, m->slots, oraw, st);
            else if (L.dim <= 32) e = launch_scan<32>(A, s->n_seqs, dec, uk, auk, m->slots, oraw, st);
            else if (L.dim <= 64) e = launch_scan<64>(A, s->n_seqs, dec, uk, auk, m->slots, oraw, st);
            else if (L.dim <= 128) e = launch_scan<128>(A, s->n_seqs, dec, uk, auk, m->slots, oraw, st);
            else e = launch_scan<256>(A, s->n_seqs, dec, uk, auk, m->slots, oraw, st);
            CU(e);
            delta_out_kernel<T><<<(Tn * L.heads + 3) / 4, 128, 0, st>>>(A, oraw, mix);
            m->launches += 3;
            mix_cols = L.heads * L.dim;
        }
        CU(linear<T>(m, mix_in, static_cast<const T*>(L.w_out), y, Tn, D, mix_cols, st));
        if (own_proj) CU(linear<T>(m, mix2, static_cast<const T*>(L.side->w_out), y2, Tn, D, mix_cols_of(*L.side), st));
        const bool last = n + 1 == m->runs.size();
        const float* next_norm1 = last ? nullptr : m->layers[m->runs[n + 1].layer].norm1;
        // the feed-forward reads hn and leaves its output in y (routed experts under the post-norm block: in `routed`)
        RoutedSum routed;
        routed.yp = nullptr; routed.slot_of = nullptr; routed.sel_w = nullptr; routed.top = 0;
        const RoutedSum no_sum = routed;
        auto actp_of = [](const SmolLmLayer& M) { return ActParams{M.mlp_act, M.act_limit, M.act_alpha, 0}; };
        // the experts (and a shared expert) of a routed feed-forward may lack gate rows
        auto expert_actp = [](const SmolLmLayer& M) { return ActParams{M.mlp_act, M.act_limit, M.act_alpha, M.ff_plain ? 1 : 0}; };
        auto feed_forward = [&]() -> int {
            if (L.mlp == SMOL_LM_MLP_POLYNORM) {
                CU(linear<T>(m, hn, static_cast<const T*>(L.w_up), z, Tn, L.ff, D, st));
                polynorm_kernel<T><<<Tn, 256, 0, st>>>(z, L.act, c.norm_eps, L.ff, act);
                CU(linear<T>(m, act, static_cast<const T*>(L.w_down), y, Tn, D, L.ff, st));
                m->launches += 1;
            } else if (L.mlp == SMOL_LM_MLP_GATED) {
                CU(linear<T>(m, hn, static_cast<const T*>(L.w_up), z, Tn, 2 * L.ff, D, st));
                gated_act_kernel<T><<<cast_grid((size_t)Tn * L.ff / 4), 256, 0, st>>>(z, L.ff, actp_of(L), (size_t)Tn, act);
                CU(linear<T>(m, act, static_cast<const T*>(L.w_down), y, Tn, D, L.ff, st));
                m->launches += 1;
            } else if (L.mlp == SMOL_LM_MLP_EXPERTS) {
                int32_t* sel_id = reinterpret_cast<int32_t*>(m->ws + m->o_sel_id);
                float* sel_w = reinterpret_cast<float*>(m->ws + m->o_sel_w);
                int32_t* perm = reinterpret_cast<int32_t*>(m->ws + m->o_perm);
                int32_t* slot_of = reinterpret_cast<int32_t*>(m->ws + m->o_slot_of);
                int32_t* seg = reinterpret_cast<int32_t*>(m->ws + m->o_seg);
                int32_t* tile_g = reinterpret_cast<int32_t*>(m->ws + m->o_tile_g);
                int32_t* tile_r = reinterpret_cast<int32_t*>(m->ws + m->o_tile_r);
                int32_t* n_tiles = reinterpret_cast<int32_t*>(m->ws + m->o_ntiles);
                float* zp = reinterpret_cast<float*>(m->ws + m->o_zp);
                T* actp = reinterpret_cast<T*>(m->ws + m->o_actp);
                float* yp = reinterpret_cast<float*>(m->ws + m->o_yp);
                RouteArgs Rt;
                Rt.w_router = L.w_router; Rt.bias = L.route_bias; Rt.D = D; Rt.E = L.n_experts + L.n_identity; Rt.E_real = L.n_experts;
                Rt.top = L.top_k; Rt.n_groups = L.n_groups; Rt.keep = L.keep_groups; Rt.scale = L.router_scale; Rt.n_tokens = Tn;
                Rt.score = L.router_score; Rt.plain = L.router_plain; Rt.group_top = L.group_rank_top;
                const int pairs = Tn * L.top_k;
                // the router reads the sublayer's input in fp32 where the block keeps it (post-norm), else its T form
                float* r_logits = reinterpret_cast<float*>(m->ws + m->o_rlogits);
                int32_t* r_done = reinterpret_cast<int32_t*>(m->ws + m->o_rdone);
                const dim3 rgrid(Tn, (Rt.E + 3) / 4);
                if (postnorm) moe_route_kernel<float><<<rgrid, 128, 0, st>>>(Rt, x, r_logits, r_done, sel_id, sel_w);
                else moe_route_kernel<T><<<rgrid, 128, 0, st>>>(Rt, hn, r_logits, r_done, sel_id, sel_w);
                m->launches += 1;
                if (L.n_experts > 0) {
                    // three forms of the two grouped products, by how many rows an expert gets: a warp per output column for
                    // a handful of pairs (decoding), 32-row mma.sync tiles, 128-row tcgen05 tiles over rows copied into sorted order
                    const int NF = L.ff_plain ? L.ff : 2 * L.ff;          // rows of an expert's first matrix
                    const bool few = !kIsF32 && pairs <= kMoeGemvPairs && D % 8 == 0 && L.ff % 8 == 0;
                    const bool big = !kIsF32 && !few && m->tc_ready && pairs / L.n_experts >= 64 && D % 8 == 0 && L.ff % 8 == 0 &&
                                     NF >= kTcTileN && D >= kTcTileN && D >= smol::umma::kBK && L.ff >= smol::umma::kBK;
                    const int tile_rows = big ? smol::umma::kM : kGroupTile;
                    moe_index_kernel<<<1, 256, 0, st>>>(sel_id, pairs, L.n_experts, tile_rows, seg, perm, slot_of, tile_g, tile_r, n_tiles);
                    const int tiles = pairs / kGroupTile + L.n_experts;
                    GemmIo io = plain_io(D, NF);
                    io.sw = (long long)NF * D;
                    io.tile_group = tile_g; io.tile_row0 = tile_r; io.seg = seg; io.n_tiles = n_tiles;
                    GemmIo io2 = plain_io(L.ff, D);
                    io2.sw = (long long)D * L.ff;
                    io2.tile_group = tile_g; io2.tile_row0 = tile_r; io2.seg = seg; io2.n_tiles = n_tiles;
                    const size_t act_n = (size_t)pairs * L.ff;
                    // a router whose weight multiplies the expert's input: the rows are copied into sorted order, each times
                    // its weight, and the products read that copy
                    T* ap = reinterpret_cast<T*>(m->ws + m->o_ap);
                    if (L.route_input) {
                        moe_gather_scaled_kernel<T><<<pairs, 128, 0, st>>>(hn, perm, L.top_k, sel_w, seg + L.n_experts, D, ap);
                        m->launches++;
                    }
                    if (few) {
                        moe_gemv_kernel<false><<<dim3((NF + 7) / 8, pairs), 256, 0, st>>>(L.route_input ? ap : hn, perm, L.route_input ? 0 : L.top_k, sel_id,
                                                                                         seg + L.n_experts, reinterpret_cast<const bf16*>(L.w_experts_in), io.sw,
                                                                                         zp, NF, D, expert_actp(L));
                        // the second product applies the activation as it reads the first one's result
                        moe_gemv_kernel<true><<<dim3((D + 7) / 8, pairs), 256, 0, st>>>(zp, perm, 0, sel_id, seg + L.n_experts,
                                                                                        reinterpret_cast<const bf16*>(L.w_experts_out), io2.sw, yp, D, L.ff, expert_actp(L));
                        m->launches += 1;
                    } else {
                        bool done = false;
                        if (big) {
                            if (!L.route_input) {
                                moe_gather_kernel<<<pairs, 128, 0, st>>>(reinterpret_cast<const bf16*>(hn), perm, L.top_k, seg + L.n_experts, D,
                                                                         reinterpret_cast<bf16*>(ap));
                                m->launches++;
                            }
                            done = linear_grouped_tc(m, reinterpret_cast<const bf16*>(ap), reinterpret_cast<const bf16*>(L.w_experts_in), zp, pairs, L.n_experts,
                                                     NF, D, io, st);
                        }
                        if (!done) {
                            if (!L.route_input) { io.gather = perm; io.gather_div = L.top_k; }
                            CU(linear_ex<T>(m, L.route_input ? ap : hn, static_cast<const T*>(L.w_experts_in), zp, pairs, NF, D, io, 1, tiles, st));
                        }
                        gated_act_kernel<T><<<cast_grid(act_n / 4), 256, 0, st>>>(zp, L.ff, expert_actp(L), (size_t)pairs, actp);
                        if (!(big && linear_grouped_tc(m, reinterpret_cast<const bf16*>(actp), reinterpret_cast<const bf16*>(L.w_experts_out), yp, pairs,
                                                       L.n_experts, D, L.ff, io2, st)))
                            CU(linear_ex<T>(m, actp, static_cast<const T*>(L.w_experts_out), yp, pairs, D, L.ff, io2, 1, tiles, st));
                    }
                    m->launches += 2;
                } else {
                    CU(cudaMemsetAsync(slot_of, 0xff, (size_t)pairs * 4, st));
                }
                if (L.shared_ff > 0) {
                    // the expert every token uses: its result lands in y and joins the routed sum in the kernel that follows
                    const int SF = L.ff_plain ? L.shared_ff : 2 * L.shared_ff;
                    CU(linear<T>(m, hn, static_cast<const T*>(L.w_shared_in), z, Tn, SF, D, st));
                    gated_act_kernel<T><<<cast_grid((size_t)Tn * L.shared_ff / 4), 256, 0, st>>>(z, L.shared_ff, expert_actp(L), (size_t)Tn, act);
                    CU(linear<T>(m, act, static_cast<const T*>(L.w_shared_out), y, Tn, D, L.shared_ff, st));
                    m->launches += 1;
                }
                // summed by the norm that follows
                routed.yp = yp; routed.slot_of = slot_of; routed.sel_w = L.route_input ? nullptr : sel_w; routed.top = L.top_k;
            }
            return SMOL_OK;
        };
        if (prenorm) {
            // x += mixer (mixers with their own projections: each normed over the width first); x += feed-forward.  The kernel
            // that ends the layer also leaves the traced row, restarts the stream where the next run asks for it and applies
            // the next layer's first norm.
            const bool has_ff = L.mlp != SMOL_LM_MLP_NONE;
            const SmolLmLayer* Ln = last ? nullptr : &m->layers[m->runs[n + 1].layer];
            const NormSpec after = Ln ? norm_of(Ln->norm1, Ln->norm1_shift, Ln->norm1_alpha) : no_norm;
            const float* restart = (!last && (m->runs[n + 1].flags & SMOL_LM_RUN_ADD_EMBED)) ? x0 : nullptr;
            float* tr_row = s->trace ? s->trace + n * (size_t)Tn * D : nullptr;
            ResidualArgs Ra;
            Ra.x = x; Ra.D = D; Ra.eps = c.norm_eps;
            Ra.y = y; Ra.y_w = own_proj ? L.proj_norm : nullptr; Ra.sy = own_proj ? L.mix_scale : 1.0f;
            Ra.y2 = own_proj ? y2 : nullptr; Ra.y2_w = own_proj ? L.side->proj_norm : nullptr; Ra.sy2 = own_proj ? L.side->mix_scale : 0.0f;
            Ra.rs = no_sum;
            Ra.trace = has_ff ? nullptr : tr_row; Ra.x0 = has_ff ? nullptr : restart;
            Ra.next = has_ff ? norm_of(L.norm2, L.norm2_shift, L.norm2_alpha) : after;
            residual_norm_kernel<T><<<Tn, nthr, D * sizeof(float), st>>>(Ra, hn, hn);
            m->launches += 1;
            if (has_ff) {
                const int rc = feed_forward();
                if (rc != SMOL_OK) return rc;
                const bool summed = routed.yp != nullptr;
                Ra.y = (!summed || L.shared_ff > 0) ? y : nullptr; Ra.y_w = nullptr; Ra.sy = 1.0f;
                Ra.y2 = nullptr; Ra.y2_w = nullptr; Ra.sy2 = 0.0f;
                Ra.rs = routed;
                Ra.trace = tr_row; Ra.x0 = restart; Ra.next = after;
                residual_norm_kernel<T><<<Tn, nthr, D * sizeof(float), st>>>(Ra, hn, hn);
                m->launches += 1;
            }
        } else if (postnorm) {
            // x <- g1 * rms_divide(alpha x + mixer); x <- g2 * rms_divide(alpha x + ff); the layer's result joins the history
            // and the stream becomes the weighted sum of the history
            const bool has_ff = L.mlp != SMOL_LM_MLP_NONE;
            post_norm_kernel<T><<<Tn, nthr, 2 * D * sizeof(float), st>>>(x, y, c.residual_alpha, L.norm1, c.norm_eps, D, has_ff ? nullptr : hist,
                                                                      hist_stride, (int)n + 2, L.depth_mix, nullptr, hn, no_sum);
            m->launches += 1;
            if (has_ff) {
                const int rc = feed_forward();
                if (rc != SMOL_OK) return rc;
                post_norm_kernel<T><<<Tn, nthr, 2 * D * sizeof(float), st>>>(x, y, c.residual_alpha, L.norm2, c.norm_eps, D, hist, hist_stride,
                                                                          (int)n + 2, L.depth_mix, nullptr, hn, routed);
                m->launches += 1;
            }
        } else if (L.mlp != SMOL_LM_MLP_NONE) {
            add_norm_kernel<T><<<Tn, nthr, D * sizeof(float), st>>>(x, y, L.norm1b, L.ls1, L.norm2, c.norm_eps, D, hn, woff, L.out_bias, no_sum, hn);
            const int rc = feed_forward();
            if (rc != SMOL_OK) return rc;
            add_norm_kernel<T><<<Tn, nthr, D * sizeof(float), st>>>(x, y, L.norm2b, L.ls2, next_norm1, c.norm_eps, D, hn, woff, nullptr, routed, hn);
            m->launches += 2;
        } else {
            add_norm_kernel<T><<<Tn, nthr, D * sizeof(float), st>>>(x, y, L.norm1b, L.ls1, next_norm1, c.norm_eps, D, hn, woff, L.out_bias, no_sum, hn);
            m->launches += 1;
        }
        if (s->trace && !prenorm) CU(cudaMemcpyAsync(s->trace + n * (size_t)Tn * D, x, (size_t)Tn * D * 4, cudaMemcpyDeviceToDevice, st));
    }
    if (s->n_want > 0) {
        if (postnorm) post_norm_kernel<T><<<s->n_want, nthr, 2 * D * sizeof(float), st>>>(x, nullptr, c.logit_scale, m->g.final_norm, c.norm_eps, D, nullptr, 0, 0,
                                                                                      nullptr, s->want_rows, hw, RoutedSum{nullptr, nullptr, nullptr, 0});
        else if (prenorm) prenorm_rows_kernel<T><<<s->n_want, nthr, 0, st>>>(x, s->want_rows, norm_of(m->g.final_norm, m->g.final_norm_shift, m->g.final_norm_alpha), D, hw);
        else norm_rows_kernel<T><<<s->n_want, nthr, 0, st>>>(x, s->want_rows, m->g.final_norm, c.norm_eps, D, hw, woff);
        m->launches++;
        CU(linear<T>(m, hw, static_cast<const T*>(m->g.head), s->logits, s->n_want, c.vocab, D, st));
        if (!postnorm && c.logit_scale != 1.0f) {
            scale_kernel<<<cast_grid((size_t)s->n_want * c.vocab), 256, 0, st>>>(s->logits, c.logit_scale, (size_t)s->n_want * c.vocab);
            m->launches++;
        }
    }
    CU(cudaGetLastError());
    return SMOL_OK;
}

extern "C" int smol_lm_step(SmolLm* m, const SmolLmStep* s, void* stream) {
    if (!m || !s) return fail(SMOL_ERR_INVALID, "smol_lm_step: null argument");
    if (!m->bound) return fail(SMOL_ERR_UNBOUND, "smol_lm_step: bind weights and pools first");
    if (s->n_tokens < 1 || s->n_seqs < 1 || s->n_want < 0 || s->max_pages < 1) return fail(SMOL_ERR_INVALID, "smol_lm_step: empty step");
    if (s->n_tokens > m->cfg.max_step_tokens || s->n_seqs > m->cfg.max_step_seqs || s->n_want > m->cfg.max_want)
        return fail(SMOL_ERR_CAPACITY, "smol_lm_step: step larger than the workspace was made for");
    if (!s->tokens || !s->tok_seq || !s->tok_pos || !s->seq_start || !s->seq_pos0 || !s->seq_slot || !s->block_table ||
        (s->n_want > 0 && (!s->want_rows || !s->logits)))
        return fail(SMOL_ERR_INVALID, "smol_lm_step: null array");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!m->cfg.use_graph || s->trace || s->n_tokens > kGraphMaxTokens)
        return m->cfg.dtype == SMOL_LM_F32 ? step_impl<float>(m, s, st) : step_impl<bf16>(m, s, st);
    // The launches of a step depend on the struct's scalars and pointers only (the arrays' contents are read on the device),
    // except that max_pos matters through the number of key ranges alone.
    SmolLmStep key = *s;
    const int max_pos = s->max_pos > 0 ? std::min(s->max_pos, m->cfg.max_context - 1) : m->cfg.max_context - 1;
    key.max_pos = std::min(m->cfg.max_context - 1, (max_pos / m->split_len + 4) / 4 * 4 * m->split_len - 1);
    for (auto& g : m->graphs)
        if (memcmp(&g.key, &key, sizeof(key)) == 0) {
            CU(cudaGraphLaunch(g.exec, st));
            m->launches += g.launches;
            return SMOL_OK;
        }
    if (!m->cap_stream) CU(cudaStreamCreateWithFlags(&m->cap_stream, cudaStreamNonBlocking));
    const int64_t before = m->launches;
    CU(cudaStreamBeginCapture(m->cap_stream, cudaStreamCaptureModeThreadLocal));
    const int rc = m->cfg.dtype == SMOL_LM_F32 ? step_impl<float>(m, &key, m->cap_stream) : step_impl<bf16>(m, &key, m->cap_stream);
    cudaGraph_t graph = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(m->cap_stream, &graph);
    if (rc != SMOL_OK) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (ce != cudaSuccess) return fail(SMOL_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(ce));
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) return fail(SMOL_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(ie));
    if (m->graphs.size() >= 64) {
        cudaGraphExecDestroy(m->graphs.front().exec);
        m->graphs.erase(m->graphs.begin());
    }
    m->graphs.push_back({key, exec, m->launches - before});
    CU(cudaGraphLaunch(exec, st));
    return SMOL_OK;
}

extern "C" int smol_lm_linear(SmolLm* m, const void* d_a, const void* d_w, float* d_y, int32_t M, int32_t N, int32_t K, void* stream) {
    if (!m || !d_a || !d_w || !d_y || M < 1 || N < 1 || K < 1) return fail(SMOL_ERR_INVALID, "smol_lm_linear: bad argument");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (m->cfg.dtype == SMOL_LM_F32) CU(linear<float>(m, static_cast<const float*>(d_a), static_cast<const float*>(d_w), d_y, M, N, K, st));
    else CU(linear<bf16>(m, static_cast<const bf16*>(d_a), static_cast<const bf16*>(d_w), d_y, M, N, K, st));
    return SMOL_OK;
}

extern "C" int smol_lm_sample(SmolLm* m, const float* d_logits, int32_t rows, int32_t n, float temp, int32_t top_k, float top_p,
                              float min_p, uint64_t seed, const int32_t* d_seq_id, const int32_t* d_step, int32_t* d_out, void* stream) {
    if (!m || !d_logits || !d_out || rows < 1) return fail(SMOL_ERR_INVALID, "smol_lm_sample: bad argument");
    if (n < 1 || n > smol::kThreads * 64) return fail(SMOL_ERR_UNSUPPORTED, "smol_lm_sample: n outside [1, 32768]");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)n * sizeof(float);
    const int grid = rows < 1024 ? rows : 1024;
    if (n <= smol::kThreads * 8) {
        CU(cudaFuncSetAttribute(lm_sample_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        lm_sample_kernel<8><<<grid, smol::kThreads, smem, st>>>(d_logits, n, rows, temp, top_k, top_p, min_p, seed, d_seq_id, d_step, d_out);
    } else {
        CU(cudaFuncSetAttribute(lm_sample_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        lm_sample_kernel<64><<<grid, smol::kThreads, smem, st>>>(d_logits, n, rows, temp, top_k, top_p, min_p, seed, d_seq_id, d_step, d_out);
    }
    CU(cudaGetLastError());
    m->launches++;
    return SMOL_OK;
}
