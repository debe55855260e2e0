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
};
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

template <class T, int MAXV>
__global__ void __launch_bounds__(kSigmoidMaxHeads * 32) sigmoid_attn_kernel(const SigmoidArgs S, const T* __restrict__ qbuf,
                                                                            const T* __restrict__ pool, T* __restrict__ out) {
    extern __shared__ float sig_smem[];      // queries [H][d], weights [H][32], mixing matrix [H][H]
    const AttnArgs& A = S.a;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31, H = A.H;
    const int t = blockIdx.x;
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
