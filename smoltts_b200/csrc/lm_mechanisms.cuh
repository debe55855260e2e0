// Further mechanisms of the hybrid language-model engine (included by lm_kernels.cu after its shared helpers):
//   - the post-norm block (one gain per norm, the stream scaled before the sublayer's output is added) with the
//     depth-weighted average of all earlier layer results,
//   - latent attention (queries through a latent; one cached latent + one rotated shared key part per position),
//   - the gated linear recurrence (decay per key channel, state [dim, vdim] per head in the sequence's slot),
//   - the state-space recurrence (short causal convolution, one decay per head and step; it shares the scan with the gated
//     linear recurrence),
//   - gated feed-forwards and the routed mixture of experts (grouped choice, identity outputs; softmax or sigmoid scores,
//     weights on the experts' outputs or inputs).
// Everything here is fp32 except what is written for a matrix product (T).
#pragma once

namespace smol {
namespace lm {

__device__ __forceinline__ float gelu_tanh_(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float silu_(float z) { return z * sigmoidf_(z); }
__device__ __forceinline__ float gated_act_(int kind, float z) {
    if (kind == SMOL_LM_ACT_SILU) return silu_(z);
    if (kind == SMOL_LM_ACT_RELU_SQUARED) {
        const float r = fmaxf(z, 0.0f);
        return r * r;
    }
    return gelu_tanh_(z);
}
// A gated unit's value from its gate and up inputs.  SMOL_LM_ACT_CLAMPED: g = min(gate, limit), u = clamp(up, -limit, limit),
// g * sigmoid(alpha * g) * (u + 1); the other kinds: act(gate) * up.  `plain`: the unit has no gate rows -- a row of the
// first product holds F values (not 2 F) and the unit's value is act(value).
struct ActParams {
    int kind;
    float limit, alpha;
    int plain;
};
__device__ __forceinline__ float gated_unit_(const ActParams& a, float g, float u) {
    if (a.plain) return gated_act_(a.kind, g);
    if (a.kind == SMOL_LM_ACT_CLAMPED) {
        g = fminf(g, a.limit);
        u = fminf(fmaxf(u, -a.limit), a.limit);
        return g * sigmoidf_(a.alpha * g) * (u + 1.0f);
    }
    return gated_act_(a.kind, g) * u;
}
__device__ __forceinline__ float softplus_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
// ln(sigmoid(z)) without overflow: -(max(-z, 0) + ln(1 + exp(-|z|)))
__device__ __forceinline__ float log_sigmoid_(float z) { return -(fmaxf(-z, 0.0f) + log1pf(expf(-fabsf(z)))); }

// ---------------------------------------------------------------------------------------------------------------------
// Post-norm block.
// Embedding: X_0 = g * rms_divide(embed[token]); the stream, the first history entry and the first sublayer's input.
template <class T>
__global__ void embed_gain_norm_kernel(const int32_t* __restrict__ tokens, const T* __restrict__ embed, int D, int vocab,
                                       const float* __restrict__ gain, float eps, float* __restrict__ x, float* __restrict__ hist0,
                                       T* __restrict__ hn) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const T* e = embed + (size_t)tok * D;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = to_f<T>(e[c]);
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = gain[0] / sqrtf(ss / (float)D + eps);
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = to_f<T>(e[c]) * r;
        x[(size_t)t * D + c] = v;
        hist0[(size_t)t * D + c] = v;
        hn[(size_t)t * D + c] = from_f<T>(v);
    }
}

// x <- g * rms_divide(alpha * x + y).  Inside a layer (hist == nullptr) that is the next sublayer's input.  At the end of
// a layer the row is the layer's result: it is stored as history entry n_hist - 1, and the stream becomes
// sum_j mix[j] * history[j] over the n_hist entries (entry 0: the embedding output), summed in ascending j.
// `rows` selects rows (final norm of the wanted rows): then only hn is written, y is not read, and alpha multiplies the
// result instead (the scale of the logits, applied before the head's product).
// (RoutedSum, the sublayer's output of a routed feed-forward summed on the fly, is declared beside add_norm_kernel.)

template <class T>
__global__ void post_norm_kernel(float* __restrict__ x, const float* __restrict__ y, float alpha, const float* __restrict__ gain, float eps,
                                 int D, float* __restrict__ hist, size_t hist_stride, int n_hist, const float* __restrict__ mix,
                                 const int32_t* __restrict__ rows, T* __restrict__ hn, const RoutedSum rs) {
    extern __shared__ float row[];          // the row before the division [D], then the earlier history's weighted sum [D]
    __shared__ float red[33];
    const size_t o = (size_t)(rows ? rows[blockIdx.x] : blockIdx.x) * D, oo = (size_t)blockIdx.x * D;
    const float* __restrict__ past = hist;   // entries 0 .. n_hist - 2 are only read here, entry n_hist - 1 only written
    float* pre = row + D;
    float ss = 0.0f;
    // a routed sublayer: the token's rows and weights are the same for every column (up to 8 kept in registers)
    int slot_r[8];
    float wt_r[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const bool in = rs.yp && k < rs.top;
        slot_r[k] = in ? rs.slot_of[(size_t)blockIdx.x * rs.top + k] : -1;
        wt_r[k] = in ? rs.sel_w[(size_t)blockIdx.x * rs.top + k] : 0.0f;
    }
    if (D <= (int)blockDim.x * kRowRegs) {
        // the row in registers: every load of a stage is issued before the first use, so a lone row (decoding) waits for
        // global memory a few times, not once per element; the gain and the row's own weight are read before the reduction
        const float g0 = gain[0];
        const float m_last = (hist && !rows) ? mix[n_hist - 1] : 0.0f;
        float v[kRowRegs], pre_r[kRowRegs];
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            v[i] = c < D ? x[o + c] : 0.0f;
            pre_r[i] = 0.0f;
        }
        if (rs.yp) {
            float acc[kRowRegs];
#pragma unroll
            for (int i = 0; i < kRowRegs; ++i) acc[i] = 0.0f;
            for (int k = 0; k < rs.top; ++k) {
                const int slot = k < 8 ? slot_r[k] : rs.slot_of[(size_t)blockIdx.x * rs.top + k];
                const float wk = k < 8 ? wt_r[k] : rs.sel_w[(size_t)blockIdx.x * rs.top + k];
#pragma unroll
                for (int i = 0; i < kRowRegs; ++i) {
                    const int c = threadIdx.x + i * blockDim.x;
                    if (c < D) acc[i] = fmaf(wk, slot >= 0 ? rs.yp[(size_t)slot * D + c] : v[i], acc[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < kRowRegs; ++i) v[i] = fmaf(alpha, v[i], acc[i]);
        } else if (!rows) {
#pragma unroll
            for (int i = 0; i < kRowRegs; ++i) {
                const int c = threadIdx.x + i * blockDim.x;
                if (c < D) v[i] = fmaf(alpha, v[i], y[o + c]);
            }
        }
        if (hist && !rows) {
#pragma unroll 2
            for (int j = 0; j + 1 < n_hist; ++j) {
                const float mj = mix[j];
#pragma unroll
                for (int i = 0; i < kRowRegs; ++i) {
                    const int c = threadIdx.x + i * blockDim.x;
                    if (c < D) pre_r[i] = fmaf(mj, past[(size_t)j * hist_stride + o + c], pre_r[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) ss += v[i] * v[i];
        ss = block_sum(ss, red);
        const float r = g0 / sqrtf(ss / (float)D + eps);
#pragma unroll
        for (int i = 0; i < kRowRegs; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c >= D) continue;
            const float w = v[i] * r;
            if (rows) {
                hn[oo + c] = from_f<T>(w * alpha);
            } else if (!hist) {
                x[o + c] = w;
                hn[o + c] = from_f<T>(w);
            } else {
                hist[(size_t)(n_hist - 1) * hist_stride + o + c] = w;
                const float acc = fmaf(m_last, w, pre_r[i]);
                x[o + c] = acc;
                hn[o + c] = from_f<T>(acc);
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        if (hist && !rows) {
            // the earlier layers' share of the new stream does not depend on this row's norm: its loads go out first
            float acc = 0.0f;
#pragma unroll 4
            for (int j = 0; j + 1 < n_hist; ++j) acc = fmaf(mix[j], past[(size_t)j * hist_stride + o + c], acc);
            pre[c] = acc;
        }
        float v = x[o + c];
        if (rs.yp) {
            float acc = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (k < rs.top) acc = fmaf(wt_r[k], slot_r[k] >= 0 ? rs.yp[(size_t)slot_r[k] * D + c] : v, acc);
            for (int k = 8; k < rs.top; ++k) {
                const int slot = rs.slot_of[(size_t)blockIdx.x * rs.top + k];
                acc = fmaf(rs.sel_w[(size_t)blockIdx.x * rs.top + k], slot >= 0 ? rs.yp[(size_t)slot * D + c] : v, acc);
            }
            v = fmaf(alpha, v, acc);
        } else if (!rows) {
            v = fmaf(alpha, v, y[o + c]);
        }
        row[c] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float r = gain[0] / sqrtf(ss / (float)D + eps);
    if (rows) {
        for (int c = threadIdx.x; c < D; c += blockDim.x) hn[oo + c] = from_f<T>(row[c] * r * alpha);
        return;
    }
    if (!hist) {
        for (int c = threadIdx.x; c < D; c += blockDim.x) {
            const float v = row[c] * r;
            x[o + c] = v;
            hn[o + c] = from_f<T>(v);
        }
        return;
    }
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        const float v = row[c] * r;
        hist[(size_t)(n_hist - 1) * hist_stride + o + c] = v;
        const float acc = fmaf(mix[n_hist - 1], v, pre[c]);
        x[o + c] = acc;
        hn[o + c] = from_f<T>(acc);
    }
}

__global__ void scale_kernel(float* __restrict__ v, float scale, size_t n) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) v[i] *= scale;
}

// ---------------------------------------------------------------------------------------------------------------------
// Latent attention.  proj row layout: query latent [q_rank] | key/value latent [kv_rank] | shared rotated key [rot] | gate [H].
// A cached position is ONE row [kv_rank + rot]: the normed latent, then the rotated key part.  Attention runs in the
// latent space: head h's query is (W_uk[h]^T q_plain[h], rotate(q_rot[h])), its score against a cached row is their dot
// product, its output the softmax-weighted sum of latents, expanded by W_uv[h] afterwards -- the same numbers as
// expanding every cached latent into per-head keys and values, without ever doing so.
struct LatentArgs {
    const float* proj;
    int n_in, q_rank, kv_rank, rot, rot_pairs, H, d;  // rot_pairs: leading pairs of the rotated part that are rotated
    float eps;
    const float *q_lat_norm, *kv_lat_norm, *freq;     // freq [rot_pairs]: base^(-i / rot_pairs)
    const int32_t *tok_seq, *tok_pos, *block_table;
    int max_pages, page_size, n_pages, n_tokens;
    size_t page_elems, k_off;
    int32_t* err;
};

// pair (a, b) of a rotated vector at position pos, pair index i
__device__ __forceinline__ void rotate_pair(float a, float b, int pos, float freq, float& ra, float& rb) {
    float sn, cs;
    sincosf((float)pos * freq, &sn, &cs);
    ra = a * cs - b * sn;
    rb = b * cs + a * sn;
}

// One block per token: the normed query latent -> cq (T), the normed key/value latent and the rotated key part -> the pool.
template <class T>
__global__ void latent_prep_kernel(const LatentArgs A, T* __restrict__ cq, T* __restrict__ pool) {
    __shared__ float red[2][33];
    const int t = blockIdx.x;
    const float* row = A.proj + (size_t)t * A.n_in;
    const float* kv = row + A.q_rank;
    // the page lookup and both sums of squares start together: their loads do not wait for one another
    const int pos = A.tok_pos[t];
    const int pg = pos / A.page_size, in_pg = pos % A.page_size;
    const int page = pg < A.max_pages ? A.block_table[(size_t)A.tok_seq[t] * A.max_pages + pg] : -1;
    float sq = 0.0f, sk = 0.0f;
    for (int c = threadIdx.x; c < A.q_rank; c += blockDim.x) sq += row[c] * row[c];
    for (int c = threadIdx.x; c < A.kv_rank; c += blockDim.x) sk += kv[c] * kv[c];
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    if (l == 0) { red[0][w] = sq; red[1][w] = sk; }
    __syncthreads();
    sq = 0.0f;
    sk = 0.0f;
    for (int i = 0; i < nw; ++i) { sq += red[0][i]; sk += red[1][i]; }      // the same order in every thread
    const float rq = 1.0f / sqrtf(sq / (float)A.q_rank + A.eps);
    for (int c = threadIdx.x; c < A.q_rank; c += blockDim.x) cq[(size_t)t * A.q_rank + c] = from_f<T>(row[c] * rq * A.q_lat_norm[c]);
    if (page < 0 || page >= A.n_pages) {
        if (threadIdx.x == 0) atomicExch(A.err, 1);
        return;
    }
    T* dst = pool + (size_t)page * A.page_elems + A.k_off + (size_t)in_pg * (A.kv_rank + A.rot);
    const float rk = 1.0f / sqrtf(sk / (float)A.kv_rank + A.eps);
    for (int c = threadIdx.x; c < A.kv_rank; c += blockDim.x) dst[c] = from_f<T>(kv[c] * rk * A.kv_lat_norm[c]);
    for (int i = threadIdx.x; i < A.rot_pairs; i += blockDim.x) {
        float ra, rb;
        rotate_pair(kv[A.kv_rank + 2 * i], kv[A.kv_rank + 2 * i + 1], pos, A.freq[i], ra, rb);
        dst[A.kv_rank + 2 * i] = from_f<T>(ra);
        dst[A.kv_rank + 2 * i + 1] = from_f<T>(rb);
    }
    for (int c = 2 * A.rot_pairs + threadIdx.x; c < A.rot; c += blockDim.x) dst[A.kv_rank + c] = from_f<T>(kv[A.kv_rank + c]);
}

// The rotated part of the attention query of (token, head): the last rot coordinates of q's head (fp32 [T][H][d + rot]),
// rotated, behind the query's latent-space part in qbuf ([T][H][kv_rank + rot], which the per-head product has written).
// One warp per (token, head).
template <class T>
__global__ void latent_query_kernel(const LatentArgs A, const float* __restrict__ q, T* __restrict__ qbuf) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= A.n_tokens * A.H) return;
    const int t = unit / A.H;
    const int pos = A.tok_pos[t];
    T* dst = qbuf + (size_t)unit * (A.kv_rank + A.rot);
    const float* qr = q + (size_t)unit * (A.d + A.rot) + A.d;
    for (int i = lane; i < A.rot_pairs; i += 32) {
        float ra, rb;
        rotate_pair(qr[2 * i], qr[2 * i + 1], pos, A.freq[i], ra, rb);
        dst[A.kv_rank + 2 * i] = from_f<T>(ra);
        dst[A.kv_rank + 2 * i + 1] = from_f<T>(rb);
    }
    for (int c = 2 * A.rot_pairs + lane; c < A.rot; c += 32) dst[A.kv_rank + c] = from_f<T>(qr[c]);
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated linear recurrence.  proj row layout: q | k [H*d each] | v | gate [H*dv each] | decay-inner [rank].
//   S_t = diag(w_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t * q_scale,  w = sigmoid(z)^(1/tau), z = W2 inner + bias.
struct GlaArgs {
    const float* proj;
    int n_in, H, d, dv, rank, n_tokens;
    float q_scale, tau, eps;
    const float *decay_w2, *decay_bias, *out_norm;     // W2 transposed [rank][H*d] fp32; bias [H*d]; plain norm weight [dv]
    const int32_t *seq_start, *seq_pos0, *seq_slot;
    size_t slot_floats, state_off;
    int n_slots;
    int32_t* err;
    // Where the scan reads a token's vectors: head h takes q_src[t * q_ld + (h / qk_share) * d + i], k likewise (qk_share
    // heads share one query / key vector), v_src[t * v_ld + h * dv + j].  The gated linear recurrence reads them from proj.
    const float *q_src, *k_src, *v_src;
    int q_ld, k_ld, v_ld, qk_share;
    // SCALAR form of the scan: one decay per (token, head) head_decay[t * H + h] instead of one per key channel, and the
    // value is multiplied by head_step[t * H + h] as it enters the state.
    const float *head_decay, *head_step;
    int out_ld;                                        // row stride of the finished mixer output
    float out_scale;
};
__host__ __device__ inline void gla_sources_from_proj(GlaArgs& A) {
    A.q_src = A.proj; A.k_src = A.proj + A.H * A.d; A.v_src = A.proj + 2 * A.H * A.d;
    A.q_ld = A.k_ld = A.v_ld = A.n_in;
    A.qk_share = 1;
    A.head_decay = A.head_step = nullptr;
    A.out_ld = A.H * A.dv;
    A.out_scale = 1.0f;
}

// decay[t][c] for the H*d key channels; blockIdx.y: a slice of blockDim.x channels
__global__ void gla_prep_kernel(const GlaArgs A, float* __restrict__ decay) {
    extern __shared__ float inner[];
    const int t = blockIdx.x, HD = A.H * A.d;
    const float* row = A.proj + (size_t)t * A.n_in + 2 * HD + 2 * A.H * A.dv;
    for (int r = threadIdx.x; r < A.rank; r += blockDim.x) inner[r] = row[r];
    __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= HD) return;
    float z = A.decay_bias[c];
#pragma unroll 8
    for (int r = 0; r < A.rank; ++r) z = fmaf(A.decay_w2[(size_t)r * HD + c], inner[r], z);
    decay[(size_t)t * HD + c] = expf(log_sigmoid_(z) / A.tau);
}

// The scan.  Value columns never mix, so a head is cut into groups of CB columns, one block per (sequence, head, group);
// L adjacent lanes share a column, lane q keeping the key rows 4*(e*L + q) .. +3 of it in registers (DK >= d rows; rows
// beyond d see zero keys and queries).  q, k, w of the head and v of the block's columns come into shared memory
// kDeltaChunk tokens at a time by cp.async, the next chunk while the current one is computed.
// Lanes per column and columns per block of the scan: from 128 key rows on, 16 lanes share a column (8 state rows per
// lane: a token's chain of dependent instructions is half as long as with 8 lanes, and a head spreads over twice the blocks;
// 32 lanes gain another 3 % only).
__host__ __device__ constexpr int gla_lanes(int DK) { return DK >= 128 ? 16 : DK >= 64 ? 8 : 4; }
__host__ __device__ constexpr int gla_block_cols(int DK) { return DK * gla_lanes(DK) <= 128 ? DK : 128 / gla_lanes(DK); }
// a buffer: q | k | w as [chunk][DK] each, v [chunk][CB], then the scalar form's decay and step [chunk] each
__host__ __device__ constexpr int gla_buf_floats(int DK) { return kDeltaChunk * (3 * DK + gla_block_cols(DK) + 2); }

template <int DK, int VEC, bool SCALAR>
__device__ __forceinline__ void gla_stage(const GlaArgs& A, float* buf, int c0, int n, int h, int j0, int nc, const float* decay) {
    constexpr int CB = gla_block_cols(DK), PL = kDeltaChunk * DK;
    const int d = A.d, HD = A.H * d, dq = d / VEC, ncq = (nc + VEC - 1) / VEC, hs = h / A.qk_share;
    for (int idx = threadIdx.x; idx < n * dq; idx += blockDim.x) {
        const int tt = idx / dq, i = (idx - tt * dq) * VEC;
        float* dst = buf + tt * DK + i;
        cp_async_f<VEC>(dst, A.q_src + (size_t)(c0 + tt) * A.q_ld + hs * d + i);
        cp_async_f<VEC>(dst + PL, A.k_src + (size_t)(c0 + tt) * A.k_ld + hs * d + i);
        if (!SCALAR) cp_async_f<VEC>(dst + 2 * PL, decay + (size_t)(c0 + tt) * HD + h * d + i);
    }
    for (int idx = threadIdx.x; idx < n * ncq; idx += blockDim.x) {
        const int tt = idx / ncq, j = (idx - tt * ncq) * VEC;
        cp_async_f<VEC>(buf + 3 * PL + tt * CB + j, A.v_src + (size_t)(c0 + tt) * A.v_ld + h * A.dv + j0 + j);
    }
    if (SCALAR) {
        float* sc = buf + 3 * PL + kDeltaChunk * CB;
        for (int tt = threadIdx.x; tt < n; tt += blockDim.x) {
            cp_async_f<1>(sc + tt, A.head_decay + (size_t)(c0 + tt) * A.H + h);
            cp_async_f<1>(sc + kDeltaChunk + tt, A.head_step + (size_t)(c0 + tt) * A.H + h);
        }
    }
}

struct TrueType { static constexpr bool value = true; };
struct FalseType { static constexpr bool value = false; };

template <int DK, bool SCALAR>
__global__ void __launch_bounds__(gla_block_cols(DK) * gla_lanes(DK)) gla_scan_kernel(const GlaArgs A, const float* __restrict__ decay,
                                                                                         float* __restrict__ state_pool,
                                                                                         float* __restrict__ o_raw) {
    constexpr int L = gla_lanes(DK), CB = gla_block_cols(DK), RV = DK / L / 4, PL = kDeltaChunk * DK;
    constexpr int kBuf = gla_buf_floats(DK);
    static_assert(DK % (4 * L) == 0, "every lane owns whole 16-byte pieces");
    extern __shared__ __align__(16) float sh[];
    const int d = A.d, dv = A.dv, NS = (dv + CB - 1) / CB;
    const int group = blockIdx.x % NS, sh_id = blockIdx.x / NS;
    const int seq = sh_id / A.H, h = sh_id % A.H;
    const int j0 = group * CB;
    const int nc = min(CB, dv - j0);
    const int col = threadIdx.x / L, q = threadIdx.x % L, j = j0 + col;
    const int t0 = A.seq_start[seq], t1 = A.seq_start[seq + 1];
    const int slot = A.seq_slot[seq];
    if (slot < 0 || slot >= A.n_slots) {
        if (threadIdx.x == 0) atomicExch(A.err, 2);
        return;
    }
    // 16-byte copies need every source to start on a 16-byte boundary: d, dv and the row lengths multiples of 4
    const bool vec = (d % 4 == 0) && (dv % 4 == 0) && (A.q_ld % 4 == 0) && (A.k_ld % 4 == 0) && (A.v_ld % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(A.q_src) | reinterpret_cast<uintptr_t>(A.k_src) | reinterpret_cast<uintptr_t>(A.v_src)) % 16 == 0);
    for (int i = threadIdx.x; i < 2 * kBuf; i += blockDim.x) sh[i] = 0.0f;      // padded channels and columns stay zero for good
    __syncthreads();
    if (vec) gla_stage<DK, 4, SCALAR>(A, sh, t0, min(kDeltaChunk, t1 - t0), h, j0, nc, decay);
    else gla_stage<DK, 1, SCALAR>(A, sh, t0, min(kDeltaChunk, t1 - t0), h, j0, nc, decay);
    cp_async_commit();
    float* st = state_pool + (size_t)slot * A.slot_floats + A.state_off + (size_t)h * d * dv;
    float S[RV][4];
    const bool fresh = A.seq_pos0[seq] == 0;
#pragma unroll
    for (int e = 0; e < RV; ++e)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = 4 * (e * L + q) + x;
            S[e][x] = (!fresh && i < d && j < dv) ? st[(size_t)i * dv + j] : 0.0f;
        }
    int cur = 0;
    for (int c0 = t0; c0 < t1; c0 += kDeltaChunk, cur ^= 1) {
        const int n = min(kDeltaChunk, t1 - c0);
        cp_async_wait<0>();
        __syncthreads();                          // this chunk has landed; every thread is done with the other buffer
        if (c0 + kDeltaChunk < t1) {
            const int nn = min(kDeltaChunk, t1 - c0 - kDeltaChunk);
            if (vec) gla_stage<DK, 4, SCALAR>(A, sh + (cur ^ 1) * kBuf, c0 + kDeltaChunk, nn, h, j0, nc, decay);
            else gla_stage<DK, 1, SCALAR>(A, sh + (cur ^ 1) * kBuf, c0 + kDeltaChunk, nn, h, j0, nc, decay);
            cp_async_commit();
        }
        const float* b = sh + cur * kBuf;
        const float4* s4 = reinterpret_cast<const float4*>(b) + q;      // piece e of a vector of token tt: s4[(tt*DK)/4 + e*L]
        const float* s_v = b + 3 * PL + col;
        const float* s_sc = b + 3 * PL + kDeltaChunk * CB;      // scalar form: decay [chunk], step [chunk]
        // four tokens at a time: their state updates follow one another, their sums over the key rows are then reduced side
        // by side, so that the shuffle latency is paid once per four tokens.  FULL: the four tokens exist (no bounds checks).
        auto group = [&](const int tt, auto full) {
            constexpr bool FULL = decltype(full)::value;
            float po[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                po[u] = 0.0f;
                if (FULL || tt + u < n) {
                    const float v = SCALAR ? s_v[(tt + u) * CB] * s_sc[kDeltaChunk + tt + u] : s_v[(tt + u) * CB];
                    const float w1 = SCALAR ? s_sc[tt + u] : 0.0f;
                    float sa = 0.0f, sb = 0.0f;
#pragma unroll
                    for (int e = 0; e < RV; ++e) {
                        const float4* p = s4 + (tt + u) * (DK / 4) + e * L;
                        const float4 qv = p[0], kv = p[PL / 4], wv = SCALAR ? make_float4(w1, w1, w1, w1) : p[2 * (PL / 4)];
                        S[e][0] = fmaf(wv.x, S[e][0], kv.x * v);
                        S[e][1] = fmaf(wv.y, S[e][1], kv.y * v);
                        S[e][2] = fmaf(wv.z, S[e][2], kv.z * v);
                        S[e][3] = fmaf(wv.w, S[e][3], kv.w * v);
                        sa = fmaf(S[e][0], qv.x, sa);
                        sb = fmaf(S[e][1], qv.y, sb);
                        sa = fmaf(S[e][2], qv.z, sa);
                        sb = fmaf(S[e][3], qv.w, sb);
                    }
                    po[u] = sa + sb;
                }
            }
#pragma unroll
            for (int s = 1; s < L; s <<= 1)
#pragma unroll
                for (int u = 0; u < 4; ++u) po[u] += __shfl_xor_sync(0xffffffffu, po[u], s);
            if (q == 0 && j < dv) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (FULL || tt + u < n) o_raw[(size_t)(c0 + tt + u) * A.H * dv + h * dv + j] = po[u] * A.q_scale;
            }
        };
        if (n == kDeltaChunk) {
            // a whole chunk, unrolled: the next group's loads and updates are issued while this group's sums are reduced
#pragma unroll
            for (int tt = 0; tt < kDeltaChunk; tt += 4) group(tt, TrueType{});
        } else {
            for (int tt = 0; tt < n; tt += 4) group(tt, FalseType{});
        }
    }
#pragma unroll
    for (int e = 0; e < RV; ++e)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int i = 4 * (e * L + q) + x;
            if (i < d && j < dv) st[(size_t)i * dv + j] = S[e][x];
        }
}

// End of the mixer: each head's o divided by its root mean square over dv, times the plain weight [dv] (shared by the
// heads), times silu(gate), written in T.  One warp per (token, head).
template <class T>
__global__ void gla_out_kernel(const GlaArgs A, const float* __restrict__ o_raw, T* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= A.n_tokens * A.H) return;
    const int t = unit / A.H, h = unit % A.H, dv = A.dv, HV = A.H * dv;
    const float* o = o_raw + (size_t)t * HV + h * dv;
    const float* gate = A.proj + (size_t)t * A.n_in + 2 * A.H * A.d + HV + h * dv;
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)dv + A.eps);
    for (int c = lane; c < dv; c += 32) out[(size_t)t * A.out_ld + h * dv + c] = from_f<T>(o[c] * rs * A.out_norm[c] * silu_(gate[c]) * A.out_scale);
}

// ---------------------------------------------------------------------------------------------------------------------
// State-space recurrence.  proj row layout: gate z [H*dv] | x [H*dv] | B [G*N] | C [G*N] | dt [H]; N = d of the scan's
// arguments (the state of a head is [N, dv]), G groups of H / G heads share B and C.  The x | B | C channels pass a causal
// convolution over the sequence's positions (taps inputs, the last tap on the current token, zeros before position 0)
// and silu.  The convolution's last taps - 1 inputs live in the sequence's slot behind the states.
struct SsdArgs {
    const float* proj;        // this mixer's rows of the fused projection
    const float* bias;        // of those rows, or nullptr
    int n_in, H, dv, N, G, taps, parts, n_tokens, n_seqs;
    float eps;
    const float *conv_w, *conv_b, *dt_bias, *a_log, *skip, *out_norm;
    const int32_t *seq_start, *seq_pos0, *seq_slot, *tok_seq;
    size_t slot_floats, conv_off;      // float offset of this run's convolution inputs inside a slot: [taps - 1][channels]
    int n_slots;
    int32_t* err;
    int out_ld;
    float out_scale;
};

// Blocks (token, slice of channels): conv[t][c] = silu(b[c] + sum_k w[c][k] * in[pos - (taps-1) + k][c]); an input of an
// earlier step comes from the slot, one before the sequence's start is zero.  The block of a token's first slice also
// leaves the heads' step dt = softplus(dt + bias) and decay exp(-exp(a_log) * dt) in `head` ([T][H] decay, then [T][H] step).
__global__ void ssd_conv_kernel(const SsdArgs A, const float* __restrict__ slots, float* __restrict__ conv, float* __restrict__ head) {
    const int t = blockIdx.x, inner = A.H * A.dv, ch = inner + 2 * A.G * A.N;
    const int s = A.tok_seq[t], t0 = A.seq_start[s], pos0 = A.seq_pos0[s];
    const int r = t - t0;                      // the token's place in this step's portion
    const int slot = A.seq_slot[s];
    if (slot < 0 || slot >= A.n_slots) {
        if (threadIdx.x == 0) atomicExch(A.err, 2);
        return;
    }
    const float* before = slots + (size_t)slot * A.slot_floats + A.conv_off;      // inputs of positions pos0 - (taps-1) .. pos0 - 1
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c < ch) {
        float acc = A.conv_b[c];
        const float bc = A.bias ? A.bias[inner + c] : 0.0f;
        for (int k = 0; k < A.taps; ++k) {
            const int back = A.taps - 1 - k;       // how many positions before the token
            float v = 0.0f;
            if (back <= r) v = A.proj[(size_t)(t - back) * A.n_in + inner + c] + bc;
            else if (pos0 + r - back >= 0) v = before[(size_t)(A.taps - 1 - (back - r)) * ch + c];
            acc = fmaf(A.conv_w[(size_t)c * A.taps + k], v, acc);
        }
        conv[(size_t)t * ch + c] = silu_(acc);
    }
    for (int h = threadIdx.x; blockIdx.y == 0 && h < A.H; h += blockDim.x) {
        const float raw = A.proj[(size_t)t * A.n_in + inner + ch + h] + (A.bias ? A.bias[inner + ch + h] : 0.0f);
        const float dt = softplus_(raw + A.dt_bias[h]);
        head[(size_t)t * A.H + h] = expf(-expf(A.a_log[h]) * dt);
        head[(size_t)(A.n_tokens + t) * A.H + h] = dt;
    }
}

// After the convolution of a step the slot keeps the last taps - 1 inputs of every sequence: channel c of sequence s.  A
// thread reads all it needs of the old inputs before it writes.  (Runs inside ssd_out_kernel, after every reader of the
// old inputs.)
constexpr int kMaxTaps = 16;
__device__ __forceinline__ void ssd_conv_state_update(const SsdArgs& A, float* __restrict__ slots, int s, int c) {
    const int inner = A.H * A.dv, ch = inner + 2 * A.G * A.N, keep = A.taps - 1;
    const int t0 = A.seq_start[s], n = A.seq_start[s + 1] - t0, pos0 = A.seq_pos0[s];
    const int slot = A.seq_slot[s];
    if (slot < 0 || slot >= A.n_slots) return;
    float* st = slots + (size_t)slot * A.slot_floats + A.conv_off;
    const float bc = A.bias ? A.bias[inner + c] : 0.0f;
    float nv[kMaxTaps];
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
        if (k >= keep) break;
        const int back = keep - k;                 // new entry k is the input `back` positions before the next token
        if (back <= n) nv[k] = A.proj[(size_t)(t0 + n - back) * A.n_in + inner + c] + bc;
        else nv[k] = (pos0 + n - back >= 0) ? st[(size_t)(keep - (back - n)) * ch + c] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
        if (k >= keep) break;
        st[(size_t)k * ch + c] = nv[k];
    }
}

// End of the mixer: y = o + skip_h * x, times silu(z), divided by the root mean square of its part (the H*dv channels form
// `parts` equal parts), times out_norm, times out_scale, written in T.  Blocks (token, part); the blocks of the
// first n_seqs tokens then bring the slots' convolution inputs up to date, one sequence per token index.
template <class T>
__global__ void ssd_out_kernel(const SsdArgs A, const float* __restrict__ o_raw, const float* __restrict__ conv, T* __restrict__ out,
                               float* __restrict__ slots) {
    __shared__ float red[33];
    const int t = blockIdx.x, inner = A.H * A.dv, ch = inner + 2 * A.G * A.N, len = inner / A.parts;
    const int c0 = blockIdx.y * len;
    const float* z = A.proj + (size_t)t * A.n_in;
    // a part's values in registers where it has at most 4 per thread (all loads issued before the first use), else recomputed
    constexpr int R = 4;
    const bool in_regs = len <= (int)blockDim.x * R;
    auto value = [&](int c) {
        const float zz = z[c] + (A.bias ? A.bias[c] : 0.0f);
        return (o_raw[(size_t)t * inner + c] + A.skip[c / A.dv] * conv[(size_t)t * ch + c]) * silu_(zz);
    };
    float val[R], wt[R];
    float ss = 0.0f;
    if (in_regs) {
        float zr[R], br[R], orr[R], sr[R], cr[R];
#pragma unroll
        for (int u = 0; u < R; ++u) {
            const int c = c0 + threadIdx.x + u * blockDim.x;
            const bool in = c < c0 + len;
            zr[u] = in ? z[c] : 0.0f;
            br[u] = (in && A.bias) ? A.bias[c] : 0.0f;
            orr[u] = in ? o_raw[(size_t)t * inner + c] : 0.0f;
            sr[u] = in ? A.skip[c / A.dv] : 0.0f;
            cr[u] = in ? conv[(size_t)t * ch + c] : 0.0f;
            wt[u] = in ? A.out_norm[c] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < R; ++u) {
            val[u] = (orr[u] + sr[u] * cr[u]) * silu_(zr[u] + br[u]);
            ss = fmaf(val[u], val[u], ss);
        }
    } else {
        for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) { const float v = value(c); ss += v * v; }
    }
    ss = block_sum(ss, red);
    const float r = A.out_scale / sqrtf(ss / (float)len + A.eps);
    if (in_regs) {
#pragma unroll
        for (int u = 0; u < R; ++u) {
            const int c = c0 + threadIdx.x + u * blockDim.x;
            if (c < c0 + len) out[(size_t)t * A.out_ld + c] = from_f<T>(val[u] * r * wt[u]);
        }
    } else {
        for (int c = c0 + threadIdx.x; c < c0 + len; c += blockDim.x) out[(size_t)t * A.out_ld + c] = from_f<T>(value(c) * r * A.out_norm[c]);
    }
    if ((int)blockIdx.x < A.n_seqs && A.taps > 1)          // the parts' blocks share a sequence's channels
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < ch; c += gridDim.y * blockDim.x) ssd_conv_state_update(A, slots, blockIdx.x, c);
}

// ---------------------------------------------------------------------------------------------------------------------
// Gated feed-forward: z rows hold gate [F] | up [F]; out = the gated unit's value (act(gate) * up, or the clamped form) in T.
template <class T>
__global__ void gated_act_kernel(const float* __restrict__ z, int F, const ActParams kind, size_t rows, T* __restrict__ out) {
    const size_t ld = kind.plain ? F : 2 * F, uo = kind.plain ? 0 : F;      // plain: the "up" operand is the value itself, unused
    if (F % 4 == 0) {                      // 16-byte pieces
        const size_t n = rows * (F / 4);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
            const size_t r = i / (F / 4), c = (i - r * (F / 4)) * 4;
            const float4 g = *reinterpret_cast<const float4*>(z + r * ld + c), u = *reinterpret_cast<const float4*>(z + r * ld + uo + c);
            store4<T>(out + r * F + c, gated_unit_(kind, g.x, u.x), gated_unit_(kind, g.y, u.y), gated_unit_(kind, g.z, u.z),
                      gated_unit_(kind, g.w, u.w));
        }
        return;
    }
    const size_t n = rows * F;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / F, c = i - r * F;
        out[i] = from_f<T>(gated_unit_(kind, z[r * ld + c], z[r * ld + uo + c]));
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// Routed mixture of experts.
struct RouteArgs {
    const float *w_router, *bias;      // [E][D] fp32, [E]
    int D, E, E_real, top, n_groups, keep;
    float scale;
    int n_tokens;
    int score;        // SMOL_LM_ROUTE_*: softmax over the outputs, or a sigmoid of each
    int plain;        // 1: a chosen output's weight is its score (times scale), not divided by the chosen scores' sum
    int group_top;    // a group is ranked by the sum of its group_top best choice scores (at most 1: by its best)
};
constexpr int kMaxRouted = 1024;       // router outputs (experts + identity outputs)
constexpr int kMaxTop = 32;

// Blocks (token, group of 4 router outputs): one warp per output takes the fp32 dot product of the token's input and the
// output's router row and leaves it in `logits`.  The block that finishes a token last (a counter per token, which it
// sets back to zero) then chooses: scores s (softmax or sigmoid), choice scores s + bias (bias == nullptr: none); outputs outside the `keep` best groups (a
// group's score: its best choice score) cannot be chosen; the `top` best choice scores are chosen (ties: the lower
// index; the choices are kept in that order), their weights are the scores s over their sum, times `scale`.  Ranks are
// counted, not sorted: output e is chosen if fewer than `top` allowed outputs beat it.
template <class TI>
__global__ void __launch_bounds__(128) moe_route_kernel(const RouteArgs A, const TI* __restrict__ x, float* __restrict__ logits,
                                                        int32_t* __restrict__ done, int32_t* __restrict__ sel_id, float* __restrict__ sel_w) {
    __shared__ float s[kMaxRouted], choice[kMaxRouted], gscore[kMaxRouted];
    __shared__ float red[33];
    __shared__ float top_s[kMaxTop];
    __shared__ int last;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const TI* xr = x + (size_t)t * A.D;
    const int e0 = blockIdx.y * nw + warp;
    if (e0 < A.E) {
        const float* wr = A.w_router + (size_t)e0 * A.D;
        float acc = 0.0f;
        if (sizeof(TI) == 4 && A.D % 4 == 0) {          // rows of x and of the router start on 16-byte boundaries
            const float4* x4 = reinterpret_cast<const float4*>(xr);
            const float4* w4 = reinterpret_cast<const float4*>(wr);
#pragma unroll 4
            for (int c = lane; c < A.D / 4; c += 32) {
                const float4 a = x4[c], b = w4[c];
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
        } else {
#pragma unroll 4
            for (int c = lane; c < A.D; c += 32) acc = fmaf(to_f<TI>(xr[c]), wr[c], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[(size_t)t * A.E + e0] = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int ticket = atomicAdd(&done[t], 1);
        last = ticket == (int)gridDim.y - 1;
        if (last) done[t] = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    float mx = -INFINITY;
    for (int e = threadIdx.x; e < A.E; e += blockDim.x) {
        const float v = __ldcg(logits + (size_t)t * A.E + e);
        s[e] = v;
        mx = fmaxf(mx, v);
    }
    mx = warp_max(mx);
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < nw; ++w) mx = fmaxf(mx, red[w]);
    float sum = 0.0f;
    if (A.score == SMOL_LM_ROUTE_SOFTMAX) {
        for (int e = threadIdx.x; e < A.E; e += blockDim.x) sum += expf(s[e] - mx);
        sum = block_sum(sum, red);
    }
    for (int e = threadIdx.x; e < A.E; e += blockDim.x) {
        const float p = A.score == SMOL_LM_ROUTE_SOFTMAX ? expf(s[e] - mx) / sum : sigmoidf_(s[e]);
        s[e] = p;
        choice[e] = p + (A.bias ? A.bias[e] : 0.0f);
    }
    __syncthreads();
    const int size = A.E / A.n_groups;
    if (A.keep < A.n_groups) {
        for (int g = threadIdx.x; g < A.n_groups; g += blockDim.x) {
            float gs = -INFINITY;
            if (A.group_top <= 1) {
                for (int e = g * size; e < (g + 1) * size; ++e) gs = fmaxf(gs, choice[e]);
            } else {
                // the scores that fewer than group_top others of the group beat (ties: the lower index first), in index order
                gs = 0.0f;
                for (int e = g * size; e < (g + 1) * size; ++e) {
                    int better = 0;
                    for (int f = g * size; f < (g + 1) * size; ++f) better += (choice[f] > choice[e] || (choice[f] == choice[e] && f < e)) ? 1 : 0;
                    if (better < A.group_top) gs += choice[e];
                }
            }
            gscore[g] = gs;
        }
        __syncthreads();
        // a group is kept if fewer than `keep` groups beat it (a higher score, or the same score and a lower index)
        for (int g = threadIdx.x; g < A.n_groups; g += blockDim.x) {
            const float gs = gscore[g];
            int better = 0;
            for (int h = 0; h < A.n_groups; ++h) better += (gscore[h] > gs || (gscore[h] == gs && h < g)) ? 1 : 0;
            if (better >= A.keep)
                for (int e = g * size; e < (g + 1) * size; ++e) choice[e] = -INFINITY;
        }
        __syncthreads();
    }
    for (int e = threadIdx.x; e < A.E; e += blockDim.x) {
        const float ce = choice[e];
        if (ce == -INFINITY) continue;
        int better = 0;
        for (int f = 0; f < A.E; ++f) better += (choice[f] > ce || (choice[f] == ce && f < e)) ? 1 : 0;
        if (better < A.top) {
            sel_id[(size_t)t * A.top + better] = e;
            top_s[better] = s[e];
        }
    }
    __syncthreads();
    if (threadIdx.x < A.top) {
        float den = 0.0f;
        for (int k = 0; k < A.top; ++k) den += top_s[k];
        sel_w[(size_t)t * A.top + threadIdx.x] = A.plain ? top_s[threadIdx.x] * A.scale : top_s[threadIdx.x] / (den + 1e-20f) * A.scale;
    }
}

// One block: sorts the (token, choice) pairs of real experts by expert.  seg[e] .. seg[e+1]-1 are expert e's rows in the
// sorted order, perm[row] the pair of a row, slot_of[pair] its row (-1: an identity output); the tile table cuts every
// expert's rows into tiles of `tile_rows` for the grouped matrix products.
__global__ void __launch_bounds__(256) moe_index_kernel(const int32_t* __restrict__ sel_id, int n_pairs, int E_real, int tile_rows,
                                                        int32_t* __restrict__ seg, int32_t* __restrict__ perm, int32_t* __restrict__ slot_of,
                                                        int32_t* __restrict__ tile_group, int32_t* __restrict__ tile_row0,
                                                        int32_t* __restrict__ n_tiles) {
    __shared__ int count[kMaxRouted + 1], cursor[kMaxRouted];
    for (int e = threadIdx.x; e <= E_real; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = sel_id[p];
        if (e < E_real) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E_real; ++e) {
            const int n = count[e];
            seg[e] = at;
            cursor[e] = at;
            for (int r0 = at; r0 < at + n; r0 += tile_rows) {
                tile_group[nt] = e;
                tile_row0[nt] = r0;
                ++nt;
            }
            at += n;
        }
        seg[E_real] = at;
        *n_tiles = nt;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const int e = sel_id[p];
        int slot = -1;
        if (e < E_real) {
            slot = atomicAdd(&cursor[e], 1);
            perm[slot] = p;
        }
        slot_of[p] = slot;
    }
}

// Rows of the sorted order copied next to each other (the tcgen05 tile reads its rows through one tensor map): row r is
// the input row of pair perm[r].  One block per row; rows beyond the sorted pairs (*n_sorted) are left alone.
__global__ void moe_gather_kernel(const bf16* __restrict__ h, const int32_t* __restrict__ perm, int div, const int32_t* __restrict__ n_sorted,
                                  int D, bf16* __restrict__ out) {
    const int r = blockIdx.x;
    if (r >= *n_sorted) return;
    const bf16* src = h + (size_t)(perm[r] / div) * D;
    bf16* dst = out + (size_t)r * D;
    if (D % 8 == 0) {
        for (int c = threadIdx.x * 8; c < D; c += blockDim.x * 8) *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
    } else {
        for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = src[c];
    }
}

// The same copy for routers whose weight multiplies the expert's INPUT: row r is weight[pair] * (the pair's input row),
// the product taken in fp32 and rounded to T once.
template <class T>
__global__ void moe_gather_scaled_kernel(const T* __restrict__ h, const int32_t* __restrict__ perm, int div, const float* __restrict__ sel_w,
                                         const int32_t* __restrict__ n_sorted, int D, T* __restrict__ out) {
    const int r = blockIdx.x;
    if (r >= *n_sorted) return;
    const int pair = perm[r];
    const float w = sel_w[pair];
    const T* src = h + (size_t)(pair / div) * D;
    T* dst = out + (size_t)r * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = from_f<T>(w * to_f<T>(src[c]));
}

// The grouped product for a handful of rows (decoding): one warp per (sorted row, output column), lanes cut K into 16-byte
// pieces, the expert's weight row is streamed once.  Sorted row r belongs to pair perm[r], whose router output names the
// expert; it reads a's row perm[r] / gather_div (gather_div == 0: row r itself).  Needs K % 8 == 0 and 16-byte aligned rows.
// ACT: a is instead the fp32 result of the first product [rows][2 K] (gate | up), and the row is the gated unit's value,
// rounded to bf16 as the tile forms round it.
constexpr int kMoeGemvPairs = 32;
template <bool ACT>
__global__ void __launch_bounds__(256) moe_gemv_kernel(const void* __restrict__ a_any, const int32_t* __restrict__ perm, int gather_div,
                                                       const int32_t* __restrict__ sel_id, const int32_t* __restrict__ n_sorted,
                                                       const bf16* __restrict__ w, long long w_stride, float* __restrict__ y, int N, int K,
                                                       const ActParams act) {
    const int r = blockIdx.y;
    if (r >= *n_sorted) return;
    const int lane = threadIdx.x & 31, n = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (n >= N) return;
    const int pair = perm[r];
    const bf16* wr = w + (long long)sel_id[pair] * w_stride + (size_t)n * K;
    float acc = 0.0f;
    if (ACT) {
        const float* zr = static_cast<const float*>(a_any) + (size_t)r * (act.plain ? K : 2 * K);
        const int uo = act.plain ? 0 : K;
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 wv = ldg_stream(wr + k);
            const float4 g0 = *reinterpret_cast<const float4*>(zr + k), g1 = *reinterpret_cast<const float4*>(zr + k + 4);
            const float4 u0 = *reinterpret_cast<const float4*>(zr + uo + k), u1 = *reinterpret_cast<const float4*>(zr + uo + k + 4);
            acc = fmaf(bf16_round(gated_unit_(act, g0.x, u0.x)), bf_lo(wv.x), acc); acc = fmaf(bf16_round(gated_unit_(act, g0.y, u0.y)), bf_hi(wv.x), acc);
            acc = fmaf(bf16_round(gated_unit_(act, g0.z, u0.z)), bf_lo(wv.y), acc); acc = fmaf(bf16_round(gated_unit_(act, g0.w, u0.w)), bf_hi(wv.y), acc);
            acc = fmaf(bf16_round(gated_unit_(act, g1.x, u1.x)), bf_lo(wv.z), acc); acc = fmaf(bf16_round(gated_unit_(act, g1.y, u1.y)), bf_hi(wv.z), acc);
            acc = fmaf(bf16_round(gated_unit_(act, g1.z, u1.z)), bf_lo(wv.w), acc); acc = fmaf(bf16_round(gated_unit_(act, g1.w, u1.w)), bf_hi(wv.w), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[(size_t)r * N + n] = acc;
        return;
    }
    const bf16* ar = static_cast<const bf16*>(a_any) + (size_t)(gather_div > 0 ? pair / gather_div : r) * K;
    for (int k = lane * 8; k < K; k += 256) {
        const uint4 wv = ldg_stream(wr + k), av = ldg_v4(ar + k);
        acc = fmaf(bf_lo(av.x), bf_lo(wv.x), acc); acc = fmaf(bf_hi(av.x), bf_hi(wv.x), acc);
        acc = fmaf(bf_lo(av.y), bf_lo(wv.y), acc); acc = fmaf(bf_hi(av.y), bf_hi(wv.y), acc);
        acc = fmaf(bf_lo(av.z), bf_lo(wv.z), acc); acc = fmaf(bf_hi(av.z), bf_hi(wv.z), acc);
        acc = fmaf(bf_lo(av.w), bf_lo(wv.w), acc); acc = fmaf(bf_hi(av.w), bf_hi(wv.w), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[(size_t)r * N + n] = acc;
}

}  // namespace lm
}  // namespace smol
