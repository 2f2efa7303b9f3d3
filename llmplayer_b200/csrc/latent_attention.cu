// Attention over a cache of low-rank latents ("latent attention").
//
// Every position of a sequence keeps one row [rank + dr]: the normed latent c (rank values) from which
// each head's keys and values are linear maps (K_h = U_h c, V_h = W_h c), and one rotated key part (dr
// values) that all heads share. A head's score against a position is
//     (q_n . U_h c + q_r . k_r) * scale  =  ((U_h^T q_n) . c + q_r . k_r) * scale,
// so the key map is applied to the query once ("absorbed") and every head attends over the same rows,
// and the head's output W_h (sum_j p_j c_j) applies the value map once to the weighted latent sum.
//
//   lp_latent_prepare   per token: RMS norm of the latent, rotation of the shared key part and of the
//                       queries' rotated parts, write of the row into the paged cache
//   lp_latent_absorb    q'[t, h] = [U_h^T q_n | q_r]
//   lp_latent_attend    online-softmax attention of q' over the rows of the pages (float32 scores,
//                       weights and sums), the keys of a sequence optionally shared out over several CTAs
//   lp_latent_expand    merge of the shares, value map, output gate
//
// All arithmetic is float32; the cache and the weights may be bfloat16 or float32. Keys are visited in
// blocks of 32 aligned to absolute positions, so a position's result does not depend on how its
// sequence was cut into steps or batched (the number of shares changes only the last merge).
#include "common.cuh"

namespace {

constexpr int KEYS = 32;            // keys per block: one per lane
constexpr int WARPS = 8;

// ---------------------------------------------------------------- prepare
template <typename TKV>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int ld, int q_off, int kv_off, const float* __restrict__ gain,
                      float eps, const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                      const int* __restrict__ seq_ids, const int* __restrict__ page_table, int pt_stride,
                      float* __restrict__ q_out, TKV* __restrict__ pages, int H, int dn, int dr, int rank,
                      int page_size, __nv_bfloat16* __restrict__ latent_out, __nv_bfloat16* __restrict__ shared_out,
                      __nv_bfloat16* __restrict__ q_half, int q_half_hd, const float* __restrict__ q_sep, int ldq,
                      int interleaved, float magnitude) {
    __shared__ float cs[128], sn[128];
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = positions[t];
    const int half = rot >> 1;
    for (int i = tid; i < half; i += blockDim.x) {
        float sv, cv;
        sincosf((float)pos * inv_freq[i], &sv, &cv);
        // a rotation may come with a factor on both cosine and sine (wavelength-stretched encodings)
        sn[i] = magnitude != 1.0f ? sv * magnitude : sv;
        cs[i] = magnitude != 1.0f ? cv * magnitude : cv;
    }
    const float* row = proj + (long long)t * ld;
    const float* kv = row + kv_off;
    float ss = 0.f;
    for (int i = tid; i < rank; i += blockDim.x) ss += kv[i] * kv[i];
    ss = lp_block_sum(ss, scratch);                       // also publishes cs / sn
    const float factor = 1.0f / sqrtf(ss / (float)rank + eps);
    const int page = page_table[(long long)seq_ids[t] * pt_stride + pos / page_size];
    const int Dk = rank + dr;
    TKV* dst = pages + ((long long)page * page_size + pos % page_size) * Dk;
    for (int i = tid; i < rank; i += blockDim.x) {
        const float c = kv[i] * factor * gain[i];
        dst[i] = lp_from_float<TKV>(c);
        if (latent_out) latent_out[(long long)t * rank + i] = __float2bfloat16_rn(c);
    }
    // the shared key part: pairs (i, i + half), or neighbours (2i, 2i + 1), of its first `rot` values turn, the rest pass
    const float* kr = kv + rank;
    for (int i = tid; i < dr; i += blockDim.x) {
        float v = kr[i];
        if (interleaved) {
            if (i < rot) {
                const int pr = i >> 1;
                v = (i & 1) ? __fadd_rn(__fmul_rn(kr[i], cs[pr]), __fmul_rn(kr[i - 1], sn[pr]))
                            : __fsub_rn(__fmul_rn(kr[i], cs[pr]), __fmul_rn(kr[i + 1], sn[pr]));
            }
        } else if (i < half) v = __fsub_rn(__fmul_rn(kr[i], cs[i]), __fmul_rn(kr[i + half], sn[i]));
        else if (i < rot) v = __fadd_rn(__fmul_rn(kr[i], cs[i - half]), __fmul_rn(kr[i - half], sn[i - half]));
        dst[rank + i] = lp_from_float<TKV>(v);
        if (shared_out) shared_out[(long long)t * dr + i] = __float2bfloat16_rn(v);
    }
    // queries: head by head [dn as projected | dr with the same rotation]
    const int hd = dn + dr;
    const float* q = q_sep ? q_sep + (long long)t * ldq : row + q_off;      // queries may come from a product of their own
    float* qo = q_out + (long long)t * H * hd;
    for (int e = tid; e < H * hd; e += blockDim.x) {
        const int i = e % hd - dn;
        float v = q[e];
        if (i >= 0) {
            if (interleaved) {
                if (i < rot) {
                    const int pr = i >> 1;
                    v = (i & 1) ? __fadd_rn(__fmul_rn(q[e], cs[pr]), __fmul_rn(q[e - 1], sn[pr]))
                                : __fsub_rn(__fmul_rn(q[e], cs[pr]), __fmul_rn(q[e + 1], sn[pr]));
                }
            } else if (i < half) v = __fsub_rn(__fmul_rn(q[e], cs[i]), __fmul_rn(q[e + half], sn[i]));
            else if (i < rot) v = __fadd_rn(__fmul_rn(q[e], cs[i - half]), __fmul_rn(q[e - half], sn[i - half]));
        }
        qo[e] = v;
        if (q_half) q_half[((long long)t * H + e / hd) * q_half_hd + e % hd] = __float2bfloat16_rn(v);
    }
    if (q_half && q_half_hd > hd) {                       // heads padded with zeros to a size the attention kernels take
        const int pad = q_half_hd - hd;
        for (int e = tid; e < H * pad; e += blockDim.x)
            q_half[((long long)t * H + e / pad) * q_half_hd + hd + e % pad] = __float2bfloat16_rn(0.f);
    }
}

// ---------------------------------------------------------------- per-head keys and values of a prompt
// For steps whose sequences all start at their first token, the heads' keys and values are formed outright
// (one product with the stacked key and value maps) and laid out as pages of keys and values, so that the
// tensor-core attention of ordinary heads serves: key of head h = [its unrotated part | the shared rotated
// part], both padded with zeros to heads of hd >= dn + dr (a size the attention kernels are built for), value of
// head h likewise. kv: bfloat16 [T, H * dn + H * dv].
__global__ void __launch_bounds__(256)
latent_heads_to_pages_kernel(const __nv_bfloat16* __restrict__ kv, const __nv_bfloat16* __restrict__ shared_part,
                             const int* __restrict__ positions, const int* __restrict__ seq_ids,
                             const int* __restrict__ table, int pt_stride, const int* __restrict__ kv_len,
                             __nv_bfloat16* __restrict__ pages, int H, int dn, int dr, int dv, int page_size, int hd) {
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int seq = seq_ids[t];
    const long long page = table[(long long)seq * pt_stride + pos / page_size];
    __nv_bfloat16* kdst = pages + page * 2 * H * page_size * hd + (long long)(pos % page_size) * hd;
    __nv_bfloat16* vdst = kdst + (long long)H * page_size * hd;
    const __nv_bfloat16* row = kv + (long long)t * H * (dn + dv);
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (int e = threadIdx.x; e < H * hd; e += blockDim.x) {
        const int h = e / hd, i = e - h * hd;
        const long long at = (long long)h * page_size * hd + i;
        kdst[at] = i < dn ? row[h * dn + i] : (i < dn + dr ? shared_part[(long long)t * dr + i - dn] : zero);
        vdst[at] = i < dv ? row[H * dn + h * dv + i] : zero;
    }
    // the sequence's last token also clears the rest of its last page: the attention kernel multiplies those rows
    // by weights of zero, which only gives zero if the rows are finite
    if (pos == kv_len[seq] - 1) {
        const int rest = page_size - 1 - pos % page_size;
        for (long long e = threadIdx.x; e < (long long)H * rest * hd; e += blockDim.x) {
            const int h = (int)(e / ((long long)rest * hd));
            const long long at = (long long)h * page_size * hd + hd + (e - (long long)h * rest * hd);
            kdst[at] = zero;
            vdst[at] = zero;
        }
    }
}

// out[t, h * dv + v] = heads[t, h * hd + v] * sigmoid(gate[t, h]): the first dv features of each head, gated.
__global__ void __launch_bounds__(256)
latent_gate_heads_kernel(const __nv_bfloat16* __restrict__ heads, const float* __restrict__ gate, int ldg,
                         __nv_bfloat16* __restrict__ out, int T, int H, int hd, int dv, float* __restrict__ zero,
                         long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long n = (long long)T * H * dv;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long th = i / dv;
        const int v = (int)(i - th * dv);
        const long long t = th / H;
        const int h = (int)(th - t * H);
        float x = __bfloat162float(heads[th * hd + v]);
        if (gate) x *= 1.0f / (1.0f + expf(-gate[t * ldg + h]));
        out[i] = __float2bfloat16_rn(x);
    }
}

// ---------------------------------------------------------------- absorb
constexpr int TOK_TILE = 8;

template <typename TW>
__global__ void __launch_bounds__(128)
latent_absorb_kernel(const float* __restrict__ q, const TW* __restrict__ uk, float* __restrict__ qa, int T, int H,
                     int dn, int dr, int rank) {
    extern __shared__ float qs[];                         // [TOK_TILE][dn]
    lp_grid_release();
    lp_grid_wait();
    const int t0 = blockIdx.x * TOK_TILE, h = blockIdx.y, tid = threadIdx.x;
    const int hd = dn + dr, Dk = rank + dr;
    const int nt = min(TOK_TILE, T - t0);
    for (int e = tid; e < TOK_TILE * dn; e += blockDim.x) {
        const int i = e / dn, d = e - i * dn;
        qs[e] = i < nt ? q[((long long)(t0 + i) * H + h) * hd + d] : 0.f;
    }
    __syncthreads();
    const TW* u = uk + (long long)h * dn * rank;
    for (int r = blockIdx.z * blockDim.x + tid; r < rank; r += gridDim.z * blockDim.x) {
        float acc[TOK_TILE];
#pragma unroll
        for (int i = 0; i < TOK_TILE; ++i) acc[i] = 0.f;
#pragma unroll 16
        for (int d = 0; d < dn; ++d) {
            const float w = lp_to_float(u[(long long)d * rank + r]);
#pragma unroll
            for (int i = 0; i < TOK_TILE; ++i) acc[i] = fmaf(qs[i * dn + d], w, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < TOK_TILE; ++i)
            if (i < nt) qa[((long long)(t0 + i) * H + h) * Dk + r] = acc[i];
    }
    for (int e = blockIdx.z * blockDim.x + tid; e < nt * dr; e += gridDim.z * blockDim.x) {
        const int i = e / dr, d = e - i * dr;
        qa[((long long)(t0 + i) * H + h) * Dk + rank + d] = q[((long long)(t0 + i) * H + h) * hd + dn + d];
    }
}

// ---------------------------------------------------------------- attend
// A CTA takes ROWS = WARPS * RW consecutive (token, head) rows of one sequence (heads of a token lie
// together, so a warp's rows mostly share their causal limit) and one share of the sequence's key blocks.
// Per block of 32 keys: the rows of the block go to shared memory as float32; lane j scores key j for the
// warp's RW rows; maximum and sum are updated per row across the warp; then lane c owns columns c, c + 32,
// ... of the latent sum and adds the 32 weighted rows in increasing key order.
template <typename TKV, int RW, int NC>
__global__ void __launch_bounds__(WARPS * 32)
latent_attend_kernel(const float* __restrict__ qa, const TKV* __restrict__ pages, const int* __restrict__ page_table,
                     int pt_stride, const int* __restrict__ q_start, const int* __restrict__ kv_len,
                     float* __restrict__ part, int H, int rank, int dr, int page_size, float scale, int shares,
                     int window) {
    extern __shared__ float smem[];
    constexpr int ROWS = WARPS * RW;
    // rows of a multiple of 4 values are read four at a time (a key row's stride of Dk + 4 floats keeps the lanes'
    // 16-byte reads on distinct banks); other widths one value at a time with a stride of Dk + 1
    const int Dk = rank + dr;
    const bool vec = (Dk & 3) == 0;
    const int KS = vec ? Dk + 4 : Dk + 1;
    float* Qs = smem;                       // [ROWS][Dk]
    float* Ks = smem + ROWS * Dk;           // [KEYS][KS]
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.y, share = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int first_tok = q_start[b], n_new = q_start[b + 1] - first_tok;
    const int len = kv_len[b];
    const int rows_total = n_new * H;
    const int r0 = blockIdx.x * ROWS;
    if (r0 >= rows_total) return;
    const int n_rows = min(ROWS, rows_total - r0);
    const int first_pos = len - n_new;                    // position of the sequence's first new token
    // queries of this CTA
    for (int r = warp; r < ROWS; r += WARPS) {
        const float* src = qa + ((long long)first_tok * H + r0 + r) * Dk;
        for (int e = lane; e < Dk; e += 32) Qs[r * Dk + e] = r < n_rows ? src[e] : 0.f;
    }
    int pos_r[RW];
    float m[RW], l[RW], o[RW][NC];
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int row = r0 + warp * RW + r;
        pos_r[r] = row < rows_total ? first_pos + row / H : -1;
        m[r] = -INFINITY;
        l[r] = 0.f;
#pragma unroll
        for (int c = 0; c < NC; ++c) o[r][c] = 0.f;
    }
    const int last_pos = first_pos + (r0 + n_rows - 1) / H;          // the CTA's largest causal limit
    // the key blocks that some row of the CTA can see (up to the largest causal limit, and from the start of the
    // first row's window on) are cut into the shares
    const int cta_first_pos = first_pos + r0 / H;
    const int blk_first = window > 0 ? max(0, cta_first_pos - window + 1) / KEYS : 0;
    const int blk_end = last_pos / KEYS + 1;
    const int per = (blk_end - blk_first + shares - 1) / shares;
    const int blk_lo = blk_first + share * per;
    const int blk_hi = min(blk_lo + per, blk_end);
    const int* pt = page_table + (long long)b * pt_stride;
    for (int blk = blk_lo; blk < blk_hi; ++blk) {
        const int k0 = blk * KEYS;
        __syncthreads();                                  // the previous block has been used (and Qs is written)
        {
            // a warp brings keys warp, warp + 8, warp + 16, warp + 24 together, so that four loads are in flight per lane
            constexpr int PER = KEYS / WARPS;
            const TKV* src[PER];
#pragma unroll
            for (int u = 0; u < PER; ++u) {
                const int kp = k0 + warp + u * WARPS;
                src[u] = kp <= last_pos ? pages + ((long long)pt[kp / page_size] * page_size + kp % page_size) * Dk : nullptr;
            }
#pragma unroll 2
            for (int e = lane; e < Dk; e += 32) {
                float v[PER];
#pragma unroll
                for (int u = 0; u < PER; ++u) v[u] = src[u] ? lp_to_float(src[u][e]) : 0.f;
#pragma unroll
                for (int u = 0; u < PER; ++u) Ks[(warp + u * WARPS) * KS + e] = v[u];
            }
        }
        __syncthreads();
        int warp_last = pos_r[0];
#pragma unroll
        for (int r = 1; r < RW; ++r) warp_last = max(warp_last, pos_r[r]);
        if (warp_last < k0) continue;                                 // nothing of this block is visible to the warp
        float dot[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) dot[r] = 0.f;
        const float* kr = Ks + lane * KS;
        const float* qw = Qs + warp * RW * Dk;
        if (vec) {
#pragma unroll 2
            for (int d = 0; d < Dk; d += 4) {
                const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const float4 qv = *reinterpret_cast<const float4*>(qw + r * Dk + d);
                    dot[r] = fmaf(qv.x, kv.x, dot[r]);
                    dot[r] = fmaf(qv.y, kv.y, dot[r]);
                    dot[r] = fmaf(qv.z, kv.z, dot[r]);
                    dot[r] = fmaf(qv.w, kv.w, dot[r]);
                }
            }
        } else {
            for (int d = 0; d < Dk; ++d) {
                const float kv = kr[d];
#pragma unroll
                for (int r = 0; r < RW; ++r) dot[r] = fmaf(qw[r * Dk + d], kv, dot[r]);
            }
        }
        float p[RW];
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const bool seen = k0 + lane <= pos_r[r] && (window <= 0 || k0 + lane > pos_r[r] - window);
            const float sc = seen ? dot[r] * scale : -INFINITY;
            const float m_new = fmaxf(m[r], lp_warp_max(sc));
            float alpha = 1.f;
            p[r] = 0.f;
            if (m_new != -INFINITY) {
                p[r] = seen ? expf(sc - m_new) : 0.f;
                alpha = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
            }
            l[r] = l[r] * alpha + lp_warp_sum(p[r]);
            m[r] = m_new;
#pragma unroll
            for (int c = 0; c < NC; ++c) o[r][c] *= alpha;
        }
        for (int j = 0; j < KEYS; ++j) {
            float pj[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) pj[r] = __shfl_sync(0xffffffffu, p[r], j);
            const float* cj = Ks + j * KS;
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                const int col = lane + 32 * c;
                if (col < rank) {
                    const float cv = cj[col];
#pragma unroll
                    for (int r = 0; r < RW; ++r) o[r][c] = fmaf(pj[r], cv, o[r][c]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RW; ++r) {
        const int row = r0 + warp * RW + r;
        if (row >= rows_total) continue;
        float* dst = part + (((long long)first_tok * H + row) * shares + share) * (rank + 2);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
            const int col = lane + 32 * c;
            if (col < rank) dst[col] = o[r][c];
        }
        if (lane == 0) {
            dst[rank] = m[r];
            dst[rank + 1] = l[r];
        }
    }
}

// ---------------------------------------------------------------- merge
// The shares of one (token, head) row become one: out = [sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M) | 0 | 1],
// the form of a single share whose sum of weights is one. One CTA per row; every warp forms the weights.
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ part, int shares, float* __restrict__ out, int rank) {
    extern __shared__ float ws[];                         // [shares]
    lp_grid_release();
    lp_grid_wait();
    const int tid = threadIdx.x, lane = tid & 31;
    const int width = rank + 2;
    const float* p = part + (long long)blockIdx.x * shares * width;
    float M = -INFINITY;
    for (int s = lane; s < shares; s += 32) M = fmaxf(M, p[s * width + rank]);
    M = lp_warp_max(M);
    float L = 0.f;
    for (int s = lane; s < shares; s += 32) {
        const float ms = p[s * width + rank];
        L += ms == -INFINITY ? 0.f : p[s * width + rank + 1] * expf(ms - M);
    }
    L = lp_warp_sum(L);
    const float inv = 1.0f / L;
    if (tid < 32)
        for (int s = lane; s < shares; s += 32) {
            const float ms = p[s * width + rank];
            ws[s] = ms == -INFINITY ? 0.f : expf(ms - M) * inv;
        }
    __syncthreads();
    float* dst = out + (long long)blockIdx.x * width;
    for (int r = tid; r < rank; r += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < shares; ++s) acc = fmaf(p[(long long)s * width + r], ws[s], acc);
        dst[r] = acc;
    }
    if (tid == 0) {
        dst[rank] = 0.f;
        dst[rank + 1] = 1.f;
    }
}

// ---------------------------------------------------------------- expand
// out[t, h * dv + v] = gate(t, h) * sum_r W[h * dv + v, r] * latent[t, h, r], where latent is the merge of
// the shares: sum_s o_s e^(m_s - M) / sum_s l_s e^(m_s - M). One warp per output feature, lanes over r.
template <typename TW, typename TOut>
__global__ void __launch_bounds__(128)
latent_expand_kernel(const float* __restrict__ part, int shares, const TW* __restrict__ uv,
                     const float* __restrict__ gate, int ldg, TOut* __restrict__ out, int T, int H, int rank, int dv,
                     float* __restrict__ zero, long long zero_count) {
    extern __shared__ float ls[];                         // [TOK_TILE][rank], then [TOK_TILE][shares] weights
    __shared__ float gs[TOK_TILE];
    float* ws = ls + TOK_TILE * rank;
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int t0 = blockIdx.x * TOK_TILE, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nt = min(TOK_TILE, T - t0);
    const int width = rank + 2;
    // each share's weight e^(m_s - M) / sum_s l_s e^(m_s - M): a warp per token, lanes over shares
    for (int i = warp; i < nt; i += 4) {
        const float* p = part + ((long long)(t0 + i) * H + h) * shares * width;
        float M = -INFINITY;
        for (int s = lane; s < shares; s += 32) M = fmaxf(M, p[s * width + rank]);
        M = lp_warp_max(M);
        float L = 0.f;
        for (int s = lane; s < shares; s += 32) {
            const float ms = p[s * width + rank];
            const float e = ms == -INFINITY ? 0.f : expf(ms - M);
            ws[i * shares + s] = e;
            L += p[s * width + rank + 1] * e;
        }
        L = lp_warp_sum(L);
        const float inv = 1.0f / L;
        for (int s = lane; s < shares; s += 32) ws[i * shares + s] *= inv;
        if (lane == 0) gs[i] = gate ? 1.0f / (1.0f + expf(-gate[(long long)(t0 + i) * ldg + h])) : 1.0f;
    }
    __syncthreads();
    for (int e = tid; e < TOK_TILE * rank; e += blockDim.x) {
        const int i = e / rank, r = e - i * rank;
        float acc = 0.f;
        if (i < nt) {
            const float* p = part + ((long long)(t0 + i) * H + h) * shares * width + r;
            const float* wi = ws + i * shares;
#pragma unroll 4
            for (int s = 0; s < shares; ++s) acc = fmaf(p[(long long)s * width], wi[s], acc);
        }
        ls[e] = acc;
    }
    __syncthreads();
    for (int v = blockIdx.z * 4 + warp; v < dv; v += gridDim.z * 4) {
        const TW* w = uv + ((long long)h * dv + v) * rank;
        float acc[TOK_TILE];
#pragma unroll
        for (int i = 0; i < TOK_TILE; ++i) acc[i] = 0.f;
#pragma unroll 8
        for (int r = lane; r < rank; r += 32) {
            const float wv = lp_to_float(w[r]);
#pragma unroll
            for (int i = 0; i < TOK_TILE; ++i) acc[i] = fmaf(ls[i * rank + r], wv, acc[i]);
        }
#pragma unroll
        for (int i = 0; i < TOK_TILE; ++i) {
            const float s = lp_warp_sum(acc[i]);
            if (lane == 0 && i < nt) out[((long long)(t0 + i) * H + h) * dv + v] = lp_from_float<TOut>(s * gs[i]);
        }
    }
}

// The same for a step of few tokens, one CTA per (token, head) row: the row's shares are merged by all threads,
// then each warp forms value features of the row (lanes over the latent).
template <typename TW, typename TOut>
__global__ void __launch_bounds__(256)
latent_expand_rows_kernel(const float* __restrict__ part, int shares, const TW* __restrict__ uv,
                          const float* __restrict__ gate, int ldg, TOut* __restrict__ out, int H, int rank, int dv,
                          float* __restrict__ zero, long long zero_count) {
    extern __shared__ float ls[];                         // [rank] merged latent, then [shares] weights
    float* ws = ls + rank;
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = blockIdx.x, t = row / H, h = row - t * H;
    const int width = rank + 2;
    const float* p = part + (long long)row * shares * width;
    float M = -INFINITY;
    for (int s = lane; s < shares; s += 32) M = fmaxf(M, p[s * width + rank]);
    M = lp_warp_max(M);
    float L = 0.f;
    for (int s = lane; s < shares; s += 32) {
        const float ms = p[s * width + rank];
        L += ms == -INFINITY ? 0.f : p[s * width + rank + 1] * expf(ms - M);
    }
    L = lp_warp_sum(L);
    const float inv = 1.0f / L;
    if (warp == 0)
        for (int s = lane; s < shares; s += 32) {
            const float ms = p[s * width + rank];
            ws[s] = ms == -INFINITY ? 0.f : expf(ms - M) * inv;
        }
    __syncthreads();
    for (int r = tid; r < rank; r += blockDim.x) {
        float acc = 0.f;
#pragma unroll 8
        for (int s = 0; s < shares; ++s) acc = fmaf(p[(long long)s * width + r], ws[s], acc);
        ls[r] = acc;
    }
    __syncthreads();
    const float g = gate ? 1.0f / (1.0f + expf(-gate[(long long)t * ldg + h])) : 1.0f;
    for (int v = warp; v < dv; v += 8) {
        const TW* w = uv + ((long long)h * dv + v) * rank;
        float acc = 0.f;
#pragma unroll 8
        for (int r = lane; r < rank; r += 32) acc = fmaf(ls[r], lp_to_float(w[r]), acc);
        acc = lp_warp_sum(acc);
        if (lane == 0) out[(long long)row * dv + v] = lp_from_float<TOut>(acc * g);
    }
}

template <typename K>
int grant_shared(K kernel, size_t bytes, const char* what) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            snprintf(lp_error_text, sizeof(lp_error_text), "%s: cannot reserve %zu bytes of shared memory: %s", what, bytes,
                     cudaGetErrorString(e));
            return -1;
        }
    }
    return 0;
}


// ---------------------------------------------------------------- the queries' own latent
// out[t, i] = x[t, off + i] / sqrt(mean_i x^2 + eps) * gain[i] for the `rank` columns from `off` of the float32
// projection: where queries go through a latent of their own, its RMS norm in front of the queries' map.
template <typename TOut>
__global__ void __launch_bounds__(256)
latent_query_norm_kernel(const float* __restrict__ proj, int ld, int off, int rank, const float* __restrict__ gain, float eps,
                         TOut* __restrict__ out) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const float* x = proj + (long long)blockIdx.x * ld + off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = lp_block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)rank + eps);
    TOut* o = out + (long long)blockIdx.x * rank;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) o[i] = lp_from_float<TOut>(x[i] * f * gain[i]);
}

}  // namespace

// proj: float32 [T, ld] with the queries at q_off ([H, dn + dr]) and the latent and shared key part at kv_off
// ([rank + dr]); pages: [num_pages, page_size, rank + dr]; q_out: float32 [T, H, dn + dr]. Optional bfloat16
// copies that lie together: latent_out [T, rank], shared_out [T, dr], q_half [T, H, q_half_hd] (heads padded with
// zeros from dn + dr to q_half_hd).
extern "C" int lp_latent_prepare(const float* proj, int ld, int q_off, int kv_off, const float* gain, float eps,
                                 const float* inv_freq, int rot, const int* positions, const int* seq_ids,
                                 const int* page_table, int pt_stride, float* q_out, void* pages, int kv_dtype, int T,
                                 int H, int dn, int dr, int rank, int page_size, void* latent_out, void* shared_out,
                                 void* q_half, int q_half_hd, const float* q_sep, int ldq, int interleaved,
                                 float magnitude, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (q_sep && ldq < H * (dn + dr)) LP_REFUSE("latent_prepare: query rows of %d for %d heads of %d", ldq, H, dn + dr);
    if (H <= 0 || dn < 0 || dr < 0 || rank <= 0 || dn + dr <= 0) LP_REFUSE("latent_prepare: %d heads of %d + %d over rank %d", H, dn, dr, rank);
    if (rot < 0 || (rot & 1) || rot > dr || rot > 256) LP_REFUSE("latent_prepare: rotary width %d of %d (even, at most 256)", rot, dr);
    if (rot > 0 && !inv_freq) LP_REFUSE("latent_prepare: rotation without frequencies");
    if (page_size <= 0) LP_REFUSE("latent_prepare: page size %d", page_size);
    if (q_half && q_half_hd < dn + dr) LP_REFUSE("latent_prepare: padded heads of %d for heads of %d", q_half_hd, dn + dr);
    if (q_off < 0 || kv_off < 0 || (!q_sep && q_off + H * (dn + dr) > ld) || kv_off + rank + dr > ld)
        LP_REFUSE("latent_prepare: slices at %d and %d do not fit rows of %d", q_off, kv_off, ld);
#define LP_LAUNCH_PREP(TKV)                                                                                       \
    lp_launch(latent_prepare_kernel<TKV>, T, 256, 0, stream, proj, ld, q_off, kv_off, gain, eps, inv_freq, rot,    \
              positions, seq_ids, page_table, pt_stride, q_out, (TKV*)pages, H, dn, dr, rank, page_size,                   \
              (__nv_bfloat16*)latent_out, (__nv_bfloat16*)shared_out, (__nv_bfloat16*)q_half, q_half_hd, q_sep, ldq,    \
              interleaved, magnitude)
    if (kv_dtype == LP_F32) LP_LAUNCH_PREP(float);
    else if (kv_dtype == LP_BF16) LP_LAUNCH_PREP(__nv_bfloat16);
    else LP_REFUSE("latent_prepare: cache dtype code %d", kv_dtype);
#undef LP_LAUNCH_PREP
    return lp_check_launch("latent_prepare");
}

// q: float32 [T, H, dn + dr]; uk: [H * dn, rank]; qa: float32 [T, H, rank + dr].
extern "C" int lp_latent_absorb(const float* q, const void* uk, int w_dtype, float* qa, int T, int H, int dn, int dr,
                                int rank, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 65535 || dn < 0 || dr < 0 || rank <= 0) LP_REFUSE("latent_absorb: %d heads of %d + %d over rank %d", H, dn, dr, rank);
    dim3 grid((T + TOK_TILE - 1) / TOK_TILE, H, (rank + 127) / 128);
    const size_t smem = (size_t)TOK_TILE * (dn > 0 ? dn : 1) * sizeof(float);
    if (w_dtype == LP_F32) {
        if (grant_shared(latent_absorb_kernel<float>, smem, "latent_absorb")) return -1;
        lp_launch(latent_absorb_kernel<float>, grid, 128, smem, stream, q, (const float*)uk, qa, T, H, dn, dr, rank);
    } else if (w_dtype == LP_BF16) {
        if (grant_shared(latent_absorb_kernel<__nv_bfloat16>, smem, "latent_absorb")) return -1;
        lp_launch(latent_absorb_kernel<__nv_bfloat16>, grid, 128, smem, stream, q, (const __nv_bfloat16*)uk, qa, T, H, dn, dr, rank);
    } else LP_REFUSE("latent_absorb: weight dtype code %d", w_dtype);
    return lp_check_launch("latent_absorb");
}

constexpr int ATTEND_RW = 4;

// How many (token, head) rows one CTA of lp_latent_attend takes.
extern "C" int lp_latent_attend_rows() { return WARPS * ATTEND_RW; }

// qa: float32 [T, H, rank + dr]; part: float32 [T, H, shares, rank + 2] (unnormalised sums, maximum, sum of
// weights); q_start [B + 1], kv_len [B] (lengths after the step); max_new: most new tokens of a sequence.
extern "C" int lp_latent_attend(const float* qa, const void* pages, int kv_dtype, const int* page_table, int pt_stride,
                                const int* q_start, const int* kv_len, float* part, int B, int max_new, int H,
                                int rank, int dr, int page_size, float scale, int shares, int window,
                                cudaStream_t stream) {
    if (B <= 0 || max_new <= 0) return 0;
    if (H <= 0 || rank <= 0 || dr < 0) LP_REFUSE("latent_attend: %d heads over rank %d + %d", H, rank, dr);
    if (rank > 512) LP_REFUSE("latent_attend: rank %d (supported: up to 512)", rank);
    if (page_size <= 0 || page_size % KEYS) LP_REFUSE("latent_attend: page size %d must be a multiple of %d", page_size, KEYS);
    if (shares <= 0 || shares > 65535 || B > 65535) LP_REFUSE("latent_attend: %d shares, %d sequences", shares, B);
    constexpr int ROWS = WARPS * ATTEND_RW;
    const int Dk = rank + dr;
    const size_t smem = ((size_t)ROWS * Dk + (size_t)KEYS * (Dk + 4)) * sizeof(float);
    if (smem > 227 * 1024) LP_REFUSE("latent_attend: rows of %d values need %zu bytes of shared memory", Dk, smem);
    dim3 grid((unsigned)(((long long)max_new * H + ROWS - 1) / ROWS), B, shares);
#define LP_LAUNCH_ATTEND(TKV, NC)                                                                                    \
    do {                                                                                                             \
        if (grant_shared(latent_attend_kernel<TKV, ATTEND_RW, NC>, smem, "latent_attend")) return -1;                \
        lp_launch(latent_attend_kernel<TKV, ATTEND_RW, NC>, grid, WARPS * 32, smem, stream, qa, (const TKV*)pages,   \
                  page_table, pt_stride, q_start, kv_len, part, H, rank, dr, page_size, scale, shares, window);      \
    } while (0)
#define LP_PICK_NC(TKV)                                  \
    do {                                                 \
        if (rank <= 32) LP_LAUNCH_ATTEND(TKV, 1);        \
        else if (rank <= 64) LP_LAUNCH_ATTEND(TKV, 2);   \
        else if (rank <= 128) LP_LAUNCH_ATTEND(TKV, 4);  \
        else if (rank <= 256) LP_LAUNCH_ATTEND(TKV, 8);  \
        else LP_LAUNCH_ATTEND(TKV, 16);                  \
    } while (0)
    if (kv_dtype == LP_F32) LP_PICK_NC(float);
    else if (kv_dtype == LP_BF16) LP_PICK_NC(__nv_bfloat16);
    else LP_REFUSE("latent_attend: cache dtype code %d", kv_dtype);
#undef LP_PICK_NC
#undef LP_LAUNCH_ATTEND
    return lp_check_launch("latent_attend");
}

// part: float32 [rows, shares, rank + 2] as lp_latent_attend leaves it; out: float32 [rows, 1, rank + 2], one share.
extern "C" int lp_latent_merge(const float* part, int shares, float* out, int rows, int rank, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (shares <= 0 || rank <= 0) LP_REFUSE("latent_merge: %d shares of rank %d", shares, rank);
    lp_launch(latent_merge_kernel, rows, 128, (size_t)shares * sizeof(float), stream, part, shares, out, rank);
    return lp_check_launch("latent_merge");
}

// part: as lp_latent_attend leaves it; uv: [H * dv, rank]; gate: float32 [T, ldg] with one value per head
// (or null); out: [T, H * dv].
// zero (optional): a float32 buffer cleared on the side. Steps of at most ROWS_FORM_TOKENS tokens take the form with one
// CTA per (token, head) row.
constexpr int ROWS_FORM_TOKENS = 64;
extern "C" int lp_latent_expand(const float* part, int shares, const void* uv, int w_dtype, const float* gate, int ldg,
                                void* out, int out_dtype, int T, int H, int rank, int dv, float* zero, long long zero_count,
                                cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || H > 65535 || rank <= 0 || dv <= 0 || shares <= 0) LP_REFUSE("latent_expand: %d heads, rank %d, values of %d, %d shares", H, rank, dv, shares);
    if (T <= ROWS_FORM_TOKENS) {
        const size_t bytes = (size_t)(rank + shares) * sizeof(float);
#define LP_LAUNCH_ROWS(TW, TOut)                                                                                     \
    do {                                                                                                             \
        if (grant_shared(latent_expand_rows_kernel<TW, TOut>, bytes, "latent_expand")) return -1;                    \
        lp_launch(latent_expand_rows_kernel<TW, TOut>, T * H, 256, bytes, stream, part, shares, (const TW*)uv, gate,  \
                  ldg, (TOut*)out, H, rank, dv, zero, zero_count);                                                   \
    } while (0)
        if (w_dtype == LP_F32 && out_dtype == LP_F32) LP_LAUNCH_ROWS(float, float);
        else if (w_dtype == LP_BF16 && out_dtype == LP_BF16) LP_LAUNCH_ROWS(__nv_bfloat16, __nv_bfloat16);
        else if (w_dtype == LP_BF16 && out_dtype == LP_F32) LP_LAUNCH_ROWS(__nv_bfloat16, float);
        else if (w_dtype == LP_F32 && out_dtype == LP_BF16) LP_LAUNCH_ROWS(float, __nv_bfloat16);
        else LP_REFUSE("latent_expand: dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef LP_LAUNCH_ROWS
        return lp_check_launch("latent_expand");
    }
    // few tokens: the value columns of a head are shared out over CTAs as well (each merges the shares itself)
    const int tiles = (T + TOK_TILE - 1) / TOK_TILE;
    int vparts = 1;
    if (tiles * H < 2 * lp_sm_count()) vparts = min((dv + 15) / 16, max(1, 2 * lp_sm_count() / (tiles * H)));
    dim3 grid(tiles, H, vparts);
    const size_t smem = (size_t)TOK_TILE * (rank + shares) * sizeof(float);
#define LP_LAUNCH_EXPAND(TW, TOut)                                                                                \
    do {                                                                                                          \
        if (grant_shared(latent_expand_kernel<TW, TOut>, smem, "latent_expand")) return -1;                       \
        lp_launch(latent_expand_kernel<TW, TOut>, grid, 128, smem, stream, part, shares, (const TW*)uv, gate, ldg, \
                  (TOut*)out, T, H, rank, dv, zero, zero_count);                                                  \
    } while (0)
    if (w_dtype == LP_F32 && out_dtype == LP_F32) LP_LAUNCH_EXPAND(float, float);
    else if (w_dtype == LP_BF16 && out_dtype == LP_BF16) LP_LAUNCH_EXPAND(__nv_bfloat16, __nv_bfloat16);
    else if (w_dtype == LP_BF16 && out_dtype == LP_F32) LP_LAUNCH_EXPAND(__nv_bfloat16, float);
    else if (w_dtype == LP_F32 && out_dtype == LP_BF16) LP_LAUNCH_EXPAND(float, __nv_bfloat16);
    else LP_REFUSE("latent_expand: dtype codes w=%d out=%d", w_dtype, out_dtype);
#undef LP_LAUNCH_EXPAND
    return lp_check_launch("latent_expand");
}

// kv: bfloat16 [T, H * dn + H * dv] (every head's unrotated keys, then every head's values); shared_part: bfloat16
// [T, dr]; pages: bfloat16 [num_pages, 2, H, page_size, hd]; table: [B, pt_stride]; kv_len [B]: the sequences'
// lengths, all of whose positions are in this step.
extern "C" int lp_latent_heads_to_pages(const void* kv, const void* shared_part, const int* positions, const int* seq_ids,
                                        const int* table, int pt_stride, const int* kv_len, void* pages, int T, int H,
                                        int dn, int dr, int dv, int page_size, int hd, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dn < 0 || dr < 0 || dv <= 0 || hd < dn + dr || dv > hd)
        LP_REFUSE("latent_heads_to_pages: %d heads of %d + %d in %d, values of %d", H, dn, dr, hd, dv);
    if (page_size <= 0) LP_REFUSE("latent_heads_to_pages: page size %d", page_size);
    lp_launch(latent_heads_to_pages_kernel, T, 256, 0, stream, (const __nv_bfloat16*)kv, (const __nv_bfloat16*)shared_part,
              positions, seq_ids, table, pt_stride, kv_len, (__nv_bfloat16*)pages, H, dn, dr, dv, page_size, hd);
    return lp_check_launch("latent_heads_to_pages");
}

extern "C" int lp_latent_gate_heads(const void* heads, const float* gate, int ldg, void* out, int T, int H, int hd, int dv,
                                    float* zero, long long zero_count, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0 || dv > hd) LP_REFUSE("latent_gate_heads: %d heads of %d, values of %d", H, hd, dv);
    const long long n = (long long)T * H * dv;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    lp_launch(latent_gate_heads_kernel, (unsigned)blocks, 256, 0, stream, (const __nv_bfloat16*)heads, gate, ldg,
              (__nv_bfloat16*)out, T, H, hd, dv, zero, zero_count);
    return lp_check_launch("latent_gate_heads");
}

// proj: float32 [T, ld]; the latent's `rank` columns start at `off`; gain: float32 [rank]; out: [T, rank].
extern "C" int lp_latent_query_norm(const float* proj, int ld, int off, int rank, const float* gain, float eps, void* out,
                                    int dtype, int T, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (rank <= 0 || off < 0 || off + rank > ld) LP_REFUSE("latent_query_norm: %d columns at %d of rows of %d", rank, off, ld);
    if (dtype == LP_F32) lp_launch(latent_query_norm_kernel<float>, T, 256, 0, stream, proj, ld, off, rank, gain, eps, (float*)out);
    else if (dtype == LP_BF16) lp_launch(latent_query_norm_kernel<__nv_bfloat16>, T, 256, 0, stream, proj, ld, off, rank, gain, eps, (__nv_bfloat16*)out);
    else LP_REFUSE("latent_query_norm: dtype code %d", dtype);
    return lp_check_launch("latent_query_norm");
}
