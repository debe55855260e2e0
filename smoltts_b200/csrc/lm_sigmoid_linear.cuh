// Further mechanisms of the hybrid language-model engine (included by lm_kernels.cu after lm_mechanisms.cuh):
//   - the pre-norm block  x += sublayer(norm(x))  with an RMS or a Dynamic-Tanh norm, a stream that may restart from
//     x + embedding output, and mixers side by side that are each projected, RMS-normed over the width and summed,
//   - sigmoid attention (no softmax: weight = sigmoid(score + head bias); the heads' weight maps mixed by a matrix;
//     chunked mask; rotated, norm-divided queries and keys; the values are the key projection),
//   - the front and back ends of two linear attentions that run on the gated linear recurrence's scan: lightning
//     attention (constant decay per head) and HGRN2 (the forget gate is the decay, one minus it the key).
// Everything here is fp32 except what is written for a matrix product or into the key/value pool (T).
#pragma once

namespace smol {
namespace lm {

// ---------------------------------------------------------------------------------------------------------------------
// Norms of the pre-norm block.  RMS: v / rms(row) * w.  Dynamic Tanh: tanh(alpha v) * w + shift, element by element.
struct NormSpec {
    int kind;                         // SMOL_LM_NORM_*
    const float *w, *shift, *alpha;   // w == nullptr: no norm follows
    float eps;
};
__device__ __forceinline__ float dyt_(const NormSpec& n, float alpha, float v, int c) { return fmaf(tanhf(alpha * v), n.w[c], n.shift[c]); }

// x[t] = embed[token[t]] * scale, kept a second time in x0 (nullptr: not needed) for the passes that restart from it;
// hn = norm(x[t]).
template <class T>
__global__ void embed_prenorm_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, float scale, int D, int vocab,
                                     const NormSpec nm, float* __restrict__ x, float* __restrict__ x0, T* __restrict__ hn) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const T* e = embed + (size_t)tok * D;
    const size_t o = (size_t)t * D;
    const float alpha = nm.kind == SMOL_LM_NORM_DYT ? nm.alpha[0] : 0.0f;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = to_f<T>(e[c]) * scale;
        x[o + c] = v;
        if (x0) x0[o + c] = v;
        if (nm.kind == SMOL_LM_NORM_DYT) hn[o + c] = from_f<T>(dyt_(nm, alpha, v, c));
        ss += v * v;
    }
    if (nm.kind == SMOL_LM_NORM_DYT) return;
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)D + nm.eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) hn[o + c] = from_f<T>(x[o + c] * r * nm.w[c]);
}

// The norm of selected rows -> T (the final norm of the rows whose logits are wanted).
template <class T>
__global__ void prenorm_rows_kernel(const float* __restrict__ x, const int32_t* __restrict__ rows, const NormSpec nm, int D, T* __restrict__ out) {
    __shared__ float red[33];
    const float* xr = x + (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * D;
    const size_t o = (size_t)blockIdx.x * D;
    if (nm.kind == SMOL_LM_NORM_DYT) {
        const float alpha = nm.alpha[0];
        for (int c = threadIdx.x; c < D; c += blockDim.x) out[o + c] = from_f<T>(dyt_(nm, alpha, xr[c], c));
        return;
    }
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) ss += xr[c] * xr[c];
    ss = block_sum(ss, red);
    const float r = 1.0f / sqrtf(ss / (float)D + nm.eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) out[o + c] = from_f<T>(xr[c] * r * nm.w[c]);
}

// End of a sublayer of the pre-norm block, fused with the norm in front of the next one.  One block per row:
//   x <- x + sy * f(y) + sy2 * f2(y2) + (the routed experts' weighted sum)
// where f(y) = y, or y / rms(y) * y_w when y_w is set (mixers side by side: each projected result is normed over the width).
// `trace` then takes the row (the stream after the sublayer); x0, when set, joins x after that (the next run restarts from
// stream + embedding output); hn <- next(x).
struct ResidualArgs {
    float* x;
    int D;
    float eps;
    const float *y, *y_w, *y2, *y2_w;     // y2 == nullptr: one result only; y == nullptr: none at all
    float sy, sy2;
    RoutedSum rs;
    float* trace;
    const float* x0;
    NormSpec next;
};

template <class T>
__global__ void residual_norm_kernel(const ResidualArgs A, T* __restrict__ hn, const T* __restrict__ hin) {
    extern __shared__ float row[];
    __shared__ float red3[3][33];
    const int D = A.D;
    const size_t o = (size_t)blockIdx.x * D;
    float r1 = A.sy, r2 = A.sy2;
    if (D <= (int)blockDim.x * kRowRegs) {
        // the row in registers: every operand is loaded before the first reduction, so a lone row (decoding) waits for
        // global memory once
        const bool dyt_r = A.next.w && A.next.kind == SMOL_LM_NORM_DYT;
        const float alpha_r = dyt_r ? A.next.alpha[0] : 0.0f;
        float xv[kRowRegs], yv[kRowRegs], zv[kRowRegs], a1[kRowRegs], a2[kRowRegs], e0[kRowRegs], nw[kRowRegs], nb[kRowRegs];
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            const bool in = c < D;
            xv[i] = in ? A.x[o + c] : 0.0f;
            yv[i] = (in && A.y) ? A.y[o + c] : 0.0f;
            zv[i] = (in && A.y2) ? A.y2[o + c] : 0.0f;
            a1[i] = (in && A.y_w) ? A.y_w[c] : 1.0f;
            a2[i] = (in && A.y2_w) ? A.y2_w[c] : 1.0f;
            e0[i] = (in && A.x0) ? A.x0[o + c] : 0.0f;
            nw[i] = (in && A.next.w) ? A.next.w[c] : 0.0f;
            nb[i] = (in && dyt_r) ? A.next.shift[c] : 0.0f;
        }
        if (A.rs.yp) {
            for (int k = 0; k < A.rs.top; ++k) {
                const int slot = A.rs.slot_of[(size_t)blockIdx.x * A.rs.top + k];
                const float wk = A.rs.sel_w ? A.rs.sel_w[(size_t)blockIdx.x * A.rs.top + k] : 1.0f;
#pragma unroll
                for (int i = 0; i < kRowRegs; ++i) {
                    const int c = threadIdx.x + i * blockDim.x;
                    if (c < D) xv[i] = fmaf(wk, slot >= 0 ? A.rs.yp[(size_t)slot * D + c] : to_f<T>(hin[o + c]), xv[i]);
                }
            }
        }
        if (A.y_w || A.y2_w) {
            float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < kRowRegs; ++i) {
                s1 = fmaf(yv[i], yv[i], s1);
                s2 = fmaf(zv[i], zv[i], s2);
            }
            block_sum3(s1, s2, s3, red3);
            if (A.y_w) r1 = A.sy / sqrtf(s1 / (float)D + A.eps);
            if (A.y2_w) r2 = A.sy2 / sqrtf(s2 / (float)D + A.eps);
            __syncthreads();
        }
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c >= D) continue;
            float v = fmaf(r2 * a2[i], zv[i], fmaf(r1 * a1[i], yv[i], xv[i]));
            if (A.trace) A.trace[o + c] = v;
            v += e0[i];
            A.x[o + c] = v;
            xv[i] = v;
            ss = fmaf(v, v, ss);
            if (dyt_r) hn[o + c] = from_f<T>(fmaf(tanhf(alpha_r * v), nw[i], nb[i]));
        }
        if (!A.next.w || dyt_r) return;
        float q2 = 0.0f, q3 = 0.0f;
        block_sum3(ss, q2, q3, red3);
        const float r = 1.0f / sqrtf(ss / (float)D + A.next.eps);
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < D) hn[o + c] = from_f<T>(xv[i] * r * nw[i]);
        }
        return;
    }
    if (A.y_w || A.y2_w) {
        float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            const float a = A.y[o + c], b = A.y2 ? A.y2[o + c] : 0.0f;
            s1 = fmaf(a, a, s1);
            s2 = fmaf(b, b, s2);
        }
        block_sum3(s1, s2, s3, red3);
        if (A.y_w) r1 = A.sy / sqrtf(s1 / (float)D + A.eps);
        if (A.y2_w) r2 = A.sy2 / sqrtf(s2 / (float)D + A.eps);
        __syncthreads();
    }
    const bool dyt = A.next.w && A.next.kind == SMOL_LM_NORM_DYT;
    const float alpha = dyt ? A.next.alpha[0] : 0.0f;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float v = A.x[o + c];
        if (A.y) v = fmaf(r1 * (A.y_w ? A.y_w[c] : 1.0f), A.y[o + c], v);
        if (A.y2) v = fmaf(r2 * (A.y2_w ? A.y2_w[c] : 1.0f), A.y2[o + c], v);
        if (A.rs.yp) {
            float acc = 0.0f;
            for (int k = 0; k < A.rs.top; ++k) {
                const int slot = A.rs.slot_of[(size_t)blockIdx.x * A.rs.top + k];
                const float e = slot >= 0 ? A.rs.yp[(size_t)slot * D + c] : to_f<T>(hin[o + c]);
                acc = fmaf(A.rs.sel_w ? A.rs.sel_w[(size_t)blockIdx.x * A.rs.top + k] : 1.0f, e, acc);
            }
            v += acc;
        }
        if (A.trace) A.trace[o + c] = v;
        if (A.x0) v += A.x0[o + c];
        A.x[o + c] = v;
        if (dyt) hn[o + c] = from_f<T>(dyt_(A.next, alpha, v, c));
        else row[c] = v;
        ss = fmaf(v, v, ss);
    }
    if (!A.next.w || dyt) return;
    float s2 = 0.0f, s3 = 0.0f;
    block_sum3(ss, s2, s3, red3);
    const float r = 1.0f / sqrtf(ss / (float)D + A.next.eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) hn[o + c] = from_f<T>(row[c] * r * A.next.w[c]);
}

// ---------------------------------------------------------------------------------------------------------------------
// Sigmoid attention.  proj row layout: q [H*d] | k [G*d] | gate [H].  Uses the softmax attention's argument block (pages,
// sizes, bias, the per-head gate through gate_off / gate_step 0) with these additions.
struct SigmoidArgs {
    AttnArgs a;
    int chunk;                     // 0: every earlier key
    int rot_pairs;                 // leading pairs (2i, 2i+1) of a head that are rotated
    const float* freq;             // [rot_pairs]
    const float *head_bias, *talk; // [H], [H][H]
    int only;                      // which sequences the warp-per-head kernel serves: 0 all, 1 those of more than kShortSeq tokens, 2 the others
    // tiled kernel: the keys are cut into absolute ranges of range_len positions (a multiple of its key tile), one block per
    // (row tile, sequence, range); with more than one range the blocks leave fp32 partial sums in `partial`
    // [n_ranges][tokens][H * dv] and sigmoid_merge_kernel adds them in range order (the weights are not normalised, so
    // partial sums simply add)
    int range_len, n_ranges;
    float* partial;
};
// ranges a row tile touches: from the range of its first row's first key to the range of its last row's position
__device__ __forceinline__ int sigmoid_tile_ranges(const SigmoidArgs& S, int first_pos, int last_pos, int& r0) {
    r0 = (S.chunk > 0 ? first_pos / S.chunk * S.chunk : 0) / S.range_len;
    return last_pos / S.range_len - r0 + 1;
}
__device__ __forceinline__ int sigmoid_first_key(const SigmoidArgs& S, int pos) { return S.chunk > 0 ? pos / S.chunk * S.chunk : 0; }

// One warp per (token, slot): slots 0..H-1 prepare a query head (bias, rotation, division by the root mean square) into
// qbuf; slots H..H+G-1 a key head: the biased projection itself is the cached value, its rotated and divided form the
// cached key.  A lane owns whole pairs, so a pair is rotated where it was loaded.
template <class T>
__global__ void sigmoid_prep_kernel(const SigmoidArgs S, T* __restrict__ qbuf, T* __restrict__ pool) {
    const AttnArgs& A = S.a;
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int slots = A.H + A.G;
    if (unit >= A.n_tokens * slots) return;
    const int t = unit / slots, s = unit % slots;
    const bool is_q = s < A.H;
    const int lo = is_q ? s * A.d : A.H * A.d + (s - A.H) * A.d;
    const float* src = A.proj + (size_t)t * A.n_in + lo;
    const float* bias = A.bias ? A.bias + lo : nullptr;
    const int pos = A.tok_pos[t];
    T *dst, *vdst = nullptr;
    if (is_q) {
        dst = qbuf + ((size_t)t * A.H + s) * A.d;
    } else {
        const int pg = pos / A.page_size, in_pg = pos % A.page_size;
        const int page = pg < A.max_pages ? A.block_table[(size_t)A.tok_seq[t] * A.max_pages + pg] : -1;
        if (page < 0 || page >= A.n_pages) {
            if (lane == 0) atomicExch(A.err, 1);
            return;
        }
        T* base = pool + (size_t)page * A.page_elems;
        const int g = s - A.H;
        dst = base + A.k_off + ((size_t)g * A.page_size + in_pg) * A.d;
        vdst = base + A.v_off + ((size_t)g * A.page_size + in_pg) * A.dv;
    }
    const int pairs = (A.d + 1) / 2;
    float ss = 0.0f;
    for (int p = lane; p < pairs; p += 32) {
        const int c = 2 * p;
        const bool two = c + 1 < A.d;
        const float u = src[c] + (bias ? bias[c] : 0.0f), v = two ? src[c + 1] + (bias ? bias[c + 1] : 0.0f) : 0.0f;
        ss = fmaf(u, u, fmaf(v, v, ss));      // a rotation keeps the pair's length
    }
    ss = warp_sum(ss);
    const float r = 1.0f / sqrtf(ss / (float)A.d + A.eps);
    for (int p = lane; p < pairs; p += 32) {
        const int c = 2 * p;
        const bool two = c + 1 < A.d;
        const float u = src[c] + (bias ? bias[c] : 0.0f), v = two ? src[c + 1] + (bias ? bias[c + 1] : 0.0f) : 0.0f;
        if (vdst) {
            vdst[c] = from_f<T>(u);
            if (two) vdst[c + 1] = from_f<T>(v);
        }
        float ru = u, rv = v;
        if (p < S.rot_pairs) rotate_pair(u, v, pos, S.freq[p], ru, rv);
        dst[c] = from_f<T>(ru * r);
        if (two) dst[c + 1] = from_f<T>(rv * r);
    }
}

// One block per token, one warp per query head, 32 keys per round.  Lane j of warp g scores key j for head g and leaves
// sigmoid(score + bias_g) in shared memory; after a barrier warp h mixes the H weights of every key with row h of the
// mixing matrix and adds the weighted values of its key/value head.  Keys are walked from the first key of the
// query's chunk in absolute rounds, so a row's sum does not depend on how the step was cut.
constexpr int kSigmoidMaxHeads = 32;
constexpr int kSigmoidSmemMax = 200 * 1024;   // shared memory the tiled and the few-token kernels may ask for
constexpr int kSigmoidRanges = 6;             // most key ranges a row tile of the tiled kernel is cut into

template <class T, int MAXV>
__global__ void __launch_bounds__(kSigmoidMaxHeads * 32) sigmoid_attn_kernel(const SigmoidArgs S, const T* __restrict__ qbuf,
                                                                            const T* __restrict__ pool, T* __restrict__ out) {
    extern __shared__ float sig_smem[];      // queries [H][d], weights [H][32], mixing matrix [H][H]
    const AttnArgs& A = S.a;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, H = A.H;
    const int t = blockIdx.x;
    if (S.only) {
        const int sq = A.tok_seq[t];
        if ((A.seq_start[sq + 1] - A.seq_start[sq] <= kShortSeq) == (S.only == 1)) return;
    }
    const int g = h / (H / A.G);
    float* qs = sig_smem + h * A.d;
    float* ws = sig_smem + H * A.d;
    float* tk = ws + H * 32;
    for (int c = lane; c < A.d; c += 32) qs[c] = to_f<T>(qbuf[((size_t)t * H + h) * A.d + c]);
    for (int c = lane; c < H; c += 32) tk[h * H + c] = S.talk[h * H + c];
    const int pos = A.tok_pos[t];
    const int32_t* bt = A.block_table + (size_t)A.tok_seq[t] * A.max_pages;
    const float hb = S.head_bias[h];
    float o[MAXV];
#pragma unroll
    for (int e = 0; e < MAXV; ++e) o[e] = 0.0f;
    __syncthreads();
    for (int j0 = sigmoid_first_key(S, pos); j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float wgt = 0.0f;
        const T* vrow = nullptr;
        if (j <= pos) {
            const T* base = pool + (size_t)bt[j / A.page_size] * A.page_elems;
            const size_t in_pg = (size_t)g * A.page_size + j % A.page_size;
            vrow = base + A.v_off + in_pg * A.v_ld;
            wgt = sigmoidf_(fmaf(key_dot<T>(qs, base + A.k_off + in_pg * A.k_ld, A.d), A.scale, hb));
        }
        ws[h * 32 + lane] = wgt;
        __syncthreads();
        float mixed = 0.0f;
        for (int x = 0; x < H; ++x) mixed = fmaf(tk[h * H + x], ws[x * 32 + lane], mixed);
        const int cnt = min(32, pos - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, mixed, jj);
            const T* vr = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(vrow), jj));
#pragma unroll
            for (int e = 0; e < MAXV; ++e) {
                const int c = lane + e * 32;
                if (c < A.dv) o[e] = fmaf(pj, to_f<T>(vr[c]), o[e]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int e = 0; e < MAXV; ++e) {
        const int c = lane + e * 32;
        if (c < A.dv) out[(size_t)t * A.out_ld + h * A.dv + c] = from_f<T>(o[e] * attn_gate(A, t, h, c));
    }
}

// Sigmoid attention for sequences that bring few tokens (decoding, short portions): the keys of a row are cut into fixed
// absolute ranges of A.split_len positions, one block per (row, range) with a warp per head.  32 keys and values of every
// key/value head at a time are staged in shared memory by the whole block (rows padded by 16 bytes), so that no global
// load sits inside the score / mixing / value loops.  The weights are not normalised, so a range's result is a plain
// partial sum: it goes to A.part [row][range][H * dv] and sigmoid_short_merge_kernel adds the ranges in order and applies
// the gate.
template <class T>
__host__ __device__ inline size_t sigmoid_split_smem(int H, int G, int d, int dv) {
    const int pad = 16 / (int)sizeof(T);
    return ((size_t)H * (d + 32) + (size_t)H * H) * sizeof(float) + (size_t)G * 32 * ((d + pad) + (dv + pad)) * sizeof(T);
}

template <class T, int MAXV>
__global__ void __launch_bounds__(kSigmoidMaxHeads * 32) sigmoid_split_kernel(const SigmoidArgs S, const T* __restrict__ qbuf, const T* __restrict__ pool) {
    extern __shared__ __align__(16) unsigned char ss_raw[];
    constexpr int kPad = 16 / (int)sizeof(T);
    const AttnArgs& A = S.a;
    const int H = A.H, G = A.G;
    const int s = blockIdx.x / kShortSeq, r = blockIdx.x % kShortSeq;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    if (n > kShortSeq || r >= n) return;
    const int t = t0 + r, pos = A.tok_pos[t];
    const int j_first = sigmoid_first_key(S, pos);
    const int range = j_first / A.split_len + blockIdx.y;
    if (range * A.split_len > pos) return;
    const int j_lo = max(range * A.split_len, j_first), j_hi = min(pos, (range + 1) * A.split_len - 1);
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, g = h / (H / G);
    const int ldk = A.d + kPad, ldv = A.dv + kPad;
    float* qs = reinterpret_cast<float*>(ss_raw) + h * A.d;
    float* ws = reinterpret_cast<float*>(ss_raw) + H * A.d;
    float* tk = ws + H * 32;
    T* Ks = reinterpret_cast<T*>(tk + H * H);                 // H (d + 32 + H) floats: a multiple of 16 bytes when it matters (vec below)
    T* Vs = Ks + (size_t)G * 32 * ldk;
    const int32_t* bt = A.block_table + (size_t)s * A.max_pages;
    for (int c = lane; c < A.d; c += 32) qs[c] = to_f<T>(qbuf[((size_t)t * H + h) * A.d + c]);
    for (int c = lane; c < H; c += 32) tk[h * H + c] = S.talk[h * H + c];
    const float hb = S.head_bias[h];
    float o[MAXV];
#pragma unroll
    for (int e = 0; e < MAXV; ++e) o[e] = 0.0f;
    // whole 16-byte pieces when every cached row and every staged row starts on a 16-byte boundary
    const bool vec = (A.d * sizeof(T)) % 16 == 0 && (A.k_off * sizeof(T)) % 16 == 0 && (A.v_off * sizeof(T)) % 16 == 0 &&
                     ((size_t)H * (A.d + 32 + H) * sizeof(float)) % 16 == 0;
    const int chunks = vec ? A.d / kPad : A.d;                // dv == d
    for (int j0 = j_lo; j0 <= j_hi; j0 += 32) {
        const int cnt = min(32, j_hi - j0 + 1);
        __syncthreads();
        for (int idx = threadIdx.x; idx < G * cnt * 2 * chunks; idx += blockDim.x) {
            const int c = idx % chunks, kv = (idx / chunks) & 1, row = (idx / (2 * chunks)) % cnt, gk = idx / (2 * chunks * cnt);
            const int j = j0 + row;
            const T* base = pool + (size_t)bt[j / A.page_size] * A.page_elems;
            const size_t in_pg = (size_t)gk * A.page_size + j % A.page_size;
            const T* src = kv ? base + A.v_off + in_pg * A.v_ld : base + A.k_off + in_pg * A.k_ld;
            T* dst = kv ? Vs + ((size_t)gk * 32 + row) * ldv : Ks + ((size_t)gk * 32 + row) * ldk;
            if (vec) *reinterpret_cast<uint4*>(dst + c * kPad) = *reinterpret_cast<const uint4*>(src + c * kPad);
            else dst[c] = src[c];
        }
        __syncthreads();
        ws[h * 32 + lane] = lane < cnt ? sigmoidf_(fmaf(key_dot<T>(qs, Ks + ((size_t)g * 32 + lane) * ldk, A.d), A.scale, hb)) : 0.0f;
        __syncthreads();
        float mixed = 0.0f;
        for (int x = 0; x < H; ++x) mixed = fmaf(tk[h * H + x], ws[x * 32 + lane], mixed);
        const T* vs = Vs + (size_t)g * 32 * ldv;
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, mixed, jj);
#pragma unroll
            for (int e = 0; e < MAXV; ++e) {
                const int c = lane + e * 32;
                if (c < A.dv) o[e] = fmaf(pj, to_f<T>(vs[jj * ldv + c]), o[e]);
            }
        }
    }
    float* dst = A.part + ((size_t)blockIdx.x * A.n_splits + blockIdx.y) * (H * A.dv) + h * A.dv;
#pragma unroll
    for (int e = 0; e < MAXV; ++e) {
        const int c = lane + e * 32;
        if (c < A.dv) dst[c] = o[e];
    }
}

// One block per row of a short sequence: adds the ranges' partial sums in range order, applies the head's gate, writes T.
template <class T>
__global__ void sigmoid_short_merge_kernel(const SigmoidArgs S, T* __restrict__ out) {
    const AttnArgs& A = S.a;
    const int s = blockIdx.x / kShortSeq, r = blockIdx.x % kShortSeq;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    if (n > kShortSeq || r >= n) return;
    const int t = t0 + r, pos = A.tok_pos[t], cols = A.H * A.dv;
    const int ns = pos / A.split_len - sigmoid_first_key(S, pos) / A.split_len + 1;
    const float* src = A.part + (size_t)blockIdx.x * A.n_splits * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float acc = 0.0f;
        for (int z = 0; z < ns; ++z) acc += src[(size_t)z * cols + c];
        out[(size_t)t * A.out_ld + c] = from_f<T>(acc * attn_gate(A, t, c / A.dv, c % A.dv));
    }
}

// Sigmoid attention for prompt portions, bf16, on the tensor cores (mma.sync m16n8k16, fp32 accumulation).  One block per
// (16-row tile of a sequence's rows in this step, sequence); warp w owns the heads w, w + warps, ... (HPW of them at most).
// Keys and values of every key/value head are staged KT absolute positions at a time.  Per tile, in two phases:
//   1. every warp scores its heads' queries against the tile (Q K^T on the tensor cores), turns the scores into
//      sigmoid(score * scale + bias_h), zero outside the mask, and leaves them in shared memory in fp32;
//   2. after a barrier every warp mixes, for each of its heads, the H weight maps with its row of the mixing matrix (fp32
//      FMAs on the fragment it is about to feed), splits the result into a bf16 head and a bf16 remainder (16 mantissa bits
//      kept) and adds weights x values on the tensor cores.
// Masked keys weigh exactly zero, and tiles are absolute positions, so a row's sum does not depend on how the step was cut.
// The sigmoid uses the hardware exponential and division (relative error about 2^-21; this form serves bf16 only).
// Needs d % 8 == 0 and 16-byte aligned cached rows.  blockIdx.z is the key range (see SigmoidArgs): a chunk's last rows see
// many more keys than its first ones, and ranges spread them over the SMs.
template <int DK, int HPW, int KT>
__global__ void __launch_bounds__(512) sigmoid_flash_kernel(const SigmoidArgs S, const bf16* __restrict__ qbuf,
                                                                          const bf16* __restrict__ pool, bf16* __restrict__ out) {
    constexpr int LD = DK + 8, LDW = KT + 8;
    extern __shared__ __align__(16) unsigned char sf_smem[];
    const AttnArgs& A = S.a;
    const int H = A.H, G = A.G, d = A.d;
    bf16* Ks = reinterpret_cast<bf16*>(sf_smem);              // [G][KT][LD]
    bf16* Vs = Ks + (size_t)G * KT * LD;                      // [G][KT][LD]
    float* Ws = reinterpret_cast<float*>(Vs + (size_t)G * KT * LD);      // [H][16][LDW]
    float* tk = Ws + (size_t)H * 16 * LDW;                    // [H][H]
    const int s = blockIdx.y;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    const int tile = gridDim.x - 1 - blockIdx.x;
    if (n <= kShortSeq || tile * 16 >= n) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3, nw = blockDim.x >> 5;
    const int pos0 = A.tok_pos[t0];
    const int32_t* bt = A.block_table + (size_t)s * A.max_pages;
    const int row_a = tile * 16 + gq, row_b = row_a + 8;
    const bool in_a = row_a < n, in_b = row_b < n;
    const int i_a = pos0 + row_a, i_b = pos0 + row_b;
    const int lo_a = sigmoid_first_key(S, i_a), lo_b = sigmoid_first_key(S, i_b);
    const int last_pos = pos0 + min(n, tile * 16 + 16) - 1;
    int r0;
    const int n_ranges = sigmoid_tile_ranges(S, pos0 + tile * 16, last_pos, r0);
    if ((int)blockIdx.z >= n_ranges) return;
    const int j_start = max(sigmoid_first_key(S, pos0 + tile * 16) / KT * KT, (r0 + (int)blockIdx.z) * S.range_len);
    const int j_end = min(last_pos, (r0 + (int)blockIdx.z + 1) * S.range_len - 1);
    for (int i = threadIdx.x; i < H * H; i += blockDim.x) tk[i] = S.talk[i];
    // the queries of this warp's heads stay in registers as A fragments
    uint32_t qf[HPW][DK / 16][4];
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int g = min(warp + u * nw, H - 1);
        const bf16* qa = qbuf + ((size_t)(t0 + row_a) * H + g) * d + tq * 2;
        const bf16* qb = qbuf + ((size_t)(t0 + row_b) * H + g) * d + tq * 2;
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
            const int c = kk * 16 + tq * 2;
            qf[u][kk][0] = (in_a && c < d) ? *reinterpret_cast<const uint32_t*>(qa + kk * 16) : 0u;
            qf[u][kk][1] = (in_b && c < d) ? *reinterpret_cast<const uint32_t*>(qb + kk * 16) : 0u;
            qf[u][kk][2] = (in_a && c + 8 < d) ? *reinterpret_cast<const uint32_t*>(qa + kk * 16 + 8) : 0u;
            qf[u][kk][3] = (in_b && c + 8 < d) ? *reinterpret_cast<const uint32_t*>(qb + kk * 16 + 8) : 0u;
        }
    }
    float o[HPW][DK / 8][4];
#pragma unroll
    for (int u = 0; u < HPW; ++u)
#pragma unroll
        for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[u][nt][e] = 0.0f;
    for (int j0 = j_start; j0 <= j_end; j0 += KT) {
        __syncthreads();                       // every warp is done with the previous tile
        for (int idx = threadIdx.x; idx < G * KT * (DK / 8); idx += blockDim.x) {
            const int c8 = (idx % (DK / 8)) * 8, r = (idx / (DK / 8)) % KT, gk = idx / ((DK / 8) * KT);
            const int j = j0 + r;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = kv;
            if (j <= last_pos && c8 < d) {
                const bf16* base = pool + (size_t)bt[j / A.page_size] * A.page_elems;
                const size_t in_pg = (size_t)gk * A.page_size + j % A.page_size;
                kv = *reinterpret_cast<const uint4*>(base + A.k_off + in_pg * A.k_ld + c8);
                vv = *reinterpret_cast<const uint4*>(base + A.v_off + in_pg * A.v_ld + c8);
            }
            *reinterpret_cast<uint4*>(Ks + ((size_t)gk * KT + r) * LD + c8) = kv;
            *reinterpret_cast<uint4*>(Vs + ((size_t)gk * KT + r) * LD + c8) = vv;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < HPW; ++u) {
            const int g = warp + u * nw;
            if (g >= H) break;
            const bf16* Kt = Ks + (size_t)(g / (H / G)) * KT * LD;
            const float hb = S.head_bias[g];
            float sc[KT / 8][4];
#pragma unroll
            for (int nt = 0; nt < KT / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) sc[nt][e] = 0.0f;
#pragma unroll
            for (int kk = 0; kk < DK / 16; ++kk)
#pragma unroll
                for (int nt = 0; nt < KT / 8; ++nt) {
                    const bf16* p = Kt + (nt * 8 + gq) * LD + kk * 16 + tq * 2;
                    mma_bf16_16816(sc[nt], qf[u][kk][0], qf[u][kk][1], qf[u][kk][2], qf[u][kk][3], *reinterpret_cast<const uint32_t*>(p),
                                   *reinterpret_cast<const uint32_t*>(p + 8));
                }
#pragma unroll
            for (int nt = 0; nt < KT / 8; ++nt) {
                float wv[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j0 + nt * 8 + tq * 2 + (e & 1);
                    const bool see = e < 2 ? (in_a && j <= i_a && j >= lo_a) : (in_b && j <= i_b && j >= lo_b);
                    wv[e] = see ? __fdividef(1.0f, 1.0f + __expf(-fmaf(sc[nt][e], A.scale, hb))) : 0.0f;
                }
                float* wp = Ws + ((size_t)g * 16 + gq) * LDW + nt * 8 + tq * 2;
                *reinterpret_cast<float2*>(wp) = make_float2(wv[0], wv[1]);
                *reinterpret_cast<float2*>(wp + 8 * LDW) = make_float2(wv[2], wv[3]);
            }
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < HPW; ++u) {
            const int h = warp + u * nw;
            if (h >= H) break;
            const bf16* Vt = Vs + (size_t)(h / (H / G)) * KT * LD;
            const float* th = tk + h * H;
#pragma unroll
            for (int k2 = 0; k2 < KT / 16; ++k2) {
                float m[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) m[e] = 0.0f;
                const float* wp = Ws + (size_t)gq * LDW + k2 * 16 + tq * 2;
                for (int g = 0; g < H; ++g) {
                    const float tg = th[g];
                    const float* p = wp + (size_t)g * 16 * LDW;
                    const float2 x0 = *reinterpret_cast<const float2*>(p), x1 = *reinterpret_cast<const float2*>(p + 8 * LDW);
                    const float2 x2 = *reinterpret_cast<const float2*>(p + 8), x3 = *reinterpret_cast<const float2*>(p + 8 * LDW + 8);
                    m[0] = fmaf(tg, x0.x, m[0]); m[1] = fmaf(tg, x0.y, m[1]); m[2] = fmaf(tg, x1.x, m[2]); m[3] = fmaf(tg, x1.y, m[3]);
                    m[4] = fmaf(tg, x2.x, m[4]); m[5] = fmaf(tg, x2.y, m[5]); m[6] = fmaf(tg, x3.x, m[6]); m[7] = fmaf(tg, x3.y, m[7]);
                }
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float h0 = bf16_round(m[2 * e]), h1 = bf16_round(m[2 * e + 1]);
                    hi[e] = pack_bf16(h0, h1);
                    lo[e] = pack_bf16(m[2 * e] - h0, m[2 * e + 1] - h1);
                }
#pragma unroll
                for (int nt = 0; nt < DK / 8; ++nt) {
                    uint32_t b0, b1;
                    ldmatrix_x2_trans(b0, b1, Vt + (k2 * 16 + (lane & 15)) * LD + nt * 8);
                    mma_bf16_16816(o[u][nt], hi[0], hi[1], hi[2], hi[3], b0, b1);
                    mma_bf16_16816(o[u][nt], lo[0], lo[1], lo[2], lo[3], b0, b1);
                }
            }
        }
    }
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int h = warp + u * nw;
        if (h >= H) break;
#pragma unroll
        for (int nt = 0; nt < DK / 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = e < 2 ? row_a : row_b, c = nt * 8 + tq * 2 + (e & 1);
                if (row < n && c < A.dv) {
                    const size_t t = t0 + row;
                    if (S.n_ranges > 1) S.partial[((size_t)blockIdx.z * A.n_tokens + t) * (H * A.dv) + h * A.dv + c] = o[u][nt][e];
                    else out[t * A.out_ld + h * A.dv + c] = __float2bfloat16_rn(o[u][nt][e] * attn_gate(A, t, h, c));
                }
            }
    }
}

// Adds a row's partial sums over its key ranges in range order, applies the head's gate and writes bf16.  One block per token.
__global__ void sigmoid_merge_kernel(const SigmoidArgs S, bf16* __restrict__ out) {
    const AttnArgs& A = S.a;
    const int t = blockIdx.x, s = A.tok_seq[t];
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0;
    if (n <= kShortSeq) return;
    const int tile = (t - t0) / 16, pos0 = A.tok_pos[t0];
    int r0;
    const int nr = sigmoid_tile_ranges(S, pos0 + tile * 16, pos0 + min(n, tile * 16 + 16) - 1, r0);
    const int cols = A.H * A.dv;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float acc = 0.0f;
        for (int z = 0; z < nr; ++z) acc += S.partial[((size_t)z * A.n_tokens + t) * cols + c];
        out[(size_t)t * A.out_ld + c] = __float2bfloat16_rn(acc * attn_gate(A, t, c / A.dv, c % A.dv));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Front ends of the linear attentions that run on gla_scan_kernel.
//  LIGHTNING: proj rows q | k [H*d each] | v | gate [H*dv each]: act[t] = silu(q | k | v) (row length 2 H d + H dv); the
//    scan's per-head decay is the constant decay_h and its step 1 (head: [T][H] decays, then [T][H] steps).
//  HGRN2: proj rows q | forget [H*d each] | v [H*dv]: qv[t] = silu(q); f = lower + (1 - lower) sigmoid(forget + bias) is the
//    decay per key channel and 1 - f the key.
struct LinPrepArgs {
    const float* proj;
    int n_in, H, d, dv, n_tokens;
    const float *head_decay, *forget_bias, *forget_lower;
};

__global__ void lightning_prep_kernel(const LinPrepArgs A, float* __restrict__ act, float* __restrict__ head) {
    const int t = blockIdx.x, n = 2 * A.H * A.d + A.H * A.dv;
    const float* row = A.proj + (size_t)t * A.n_in;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) act[(size_t)t * n + c] = silu_(row[c]);
    for (int h = threadIdx.x; blockIdx.y == 0 && h < A.H; h += blockDim.x) {
        head[(size_t)t * A.H + h] = A.head_decay[h];
        head[(size_t)(A.n_tokens + t) * A.H + h] = 1.0f;
    }
}

__global__ void hgrn2_prep_kernel(const LinPrepArgs A, float* __restrict__ qv, float* __restrict__ key, float* __restrict__ decay) {
    const int t = blockIdx.x, HD = A.H * A.d;
    const float* row = A.proj + (size_t)t * A.n_in;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < HD; c += gridDim.y * blockDim.x) {
        const float lo = A.forget_lower[c];
        const float f = fmaf(1.0f - lo, sigmoidf_(row[HD + c] + A.forget_bias[c]), lo);
        qv[(size_t)t * HD + c] = silu_(row[c]);
        decay[(size_t)t * HD + c] = f;
        key[(size_t)t * HD + c] = 1.0f - f;
    }
}

// Back end: the scan's raw output [T][H*dv] divided by its root mean square over `len` channels (blocks (token, part): a
// part is a head, or all heads together), times a plain weight (w[c % w_mod]: one vector per part when w_mod = len), times
// sigmoid(proj[t][gate_off + c]) when has_gate, times out_scale, written in T.
struct LinOutArgs {
    const float* proj;
    int n_in, cols, len, w_mod, has_gate, out_ld;
    size_t gate_off;
    float eps, out_scale;
    const float* weight;
};

template <class T>
__global__ void lin_attn_out_kernel(const LinOutArgs A, const float* __restrict__ o_raw, T* __restrict__ out) {
    __shared__ float red[33];
    const int t = blockIdx.x, c0 = blockIdx.y * A.len;
    const float* o = o_raw + (size_t)t * A.cols;
    float ss = 0.0f;
    for (int c = c0 + threadIdx.x; c < c0 + A.len; c += blockDim.x) ss = fmaf(o[c], o[c], ss);
    ss = block_sum(ss, red);
    const float r = A.out_scale / sqrtf(ss / (float)A.len + A.eps);
    for (int c = c0 + threadIdx.x; c < c0 + A.len; c += blockDim.x) {
        float v = o[c] * r * A.weight[c % A.w_mod];
        if (A.has_gate) v *= sigmoidf_(A.proj[(size_t)t * A.n_in + A.gate_off + c]);
        out[(size_t)t * A.out_ld + c] = from_f<T>(v);
    }
}

}  // namespace lm
}  // namespace smol
