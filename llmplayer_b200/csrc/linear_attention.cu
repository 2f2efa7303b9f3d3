// Gated linear attention: a matrix-valued recurrent state per head with a decay per key channel.
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: [dk, dv], rows belong to key channels)
//     o_t = S_t^T q_t
//
// with a_t = sigmoid(z_t)^(1/tau) and z_t = A2 (A1 h_t) + bias (a low-rank map of the layer's input).
// The state is float32, one block per sequence (stored [H, dv, dk]), read at the start of a step and written
// back at its end; decays, their logarithms and every sum are float32.
//
//   lp_gla_decay    a[t, c] = exp(-softplus(-z[t, c]) / tau), z from the low-rank factor's output; or, for the
//                   time-mixing family, a[t, c] = exp(-exp(z[t, c])) with z = A2 tanh(A1 x_t) + bias
//   lp_token_shift  per token the blends x_t + (x_(t-1) - x_t) * mu_s that such a layer's maps read
//   lp_gla_scan     the recurrence over a step's tokens, sequence by sequence, in token order
//   lp_gla_finish   per head: RMS norm over dv (gain shared by heads), times silu(gate)
#include "common.cuh"

namespace {

// ---------------------------------------------------------------- decay
// low: float32 [T, ldl] slice with the R values A1 h; a2: [C, R]; bias: [C]; out: float32 [T, C].
template <typename TW>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ low, int ldl, const TW* __restrict__ a2, const float* __restrict__ bias,
                 float* __restrict__ out, int T, int C, int R, float inv_tau, int form) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * C;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / C;
        const int c = (int)(i - t * C);
        const float* x = low + t * ldl;
        const TW* w = a2 + (long long)c * R;
        float z = 0.f;
        if (form == 1) {
            // the time-mixing form: the factor's output passes through tanh, and the decay is exp(-exp(z))
            for (int r = 0; r < R; ++r) z = fmaf(lp_to_float(w[r]), tanhf(x[r]), z);
            z += bias ? bias[c] : 0.f;
            out[i] = expf(-expf(z));
            continue;
        }
        for (int r = 0; r < R; ++r) z = fmaf(lp_to_float(w[r]), x[r], z);
        z += bias ? bias[c] : 0.f;
        // log sigmoid(z) = -softplus(-z)
        const float sp = fmaxf(-z, 0.f) + log1pf(expf(-fabsf(z)));
        out[i] = expf(-sp * inv_tau);
    }
}

// ---------------------------------------------------------------- scan
// One CTA per (block of VT value columns, head, sequence); KP threads share JT neighbouring value columns, thread
// (column group, part) keeping the state entries of key channels part, part + KP, part + 2 KP, ... of those columns
// in registers.
// Tokens are brought to shared memory TB at a time; per token every thread decays and updates its entries,
// forms its share of o_t[j], and the KP shares meet in log2(KP) shuffles. The state is stored per head as
// [dv, dk] (a column's channels lie together), so that the threads of a column read and write whole sectors.
constexpr int TB = 16;            // tokens per round of loads

//
// Long prompts are cut into chunks of `chunk` tokens that run side by side (blockIdx.z = sequence * chunks + chunk):
//   mode LOCAL    every chunk starts from zero, writes no output, and leaves its final state and the product of its
//                 decays per channel in `chunk_state` / `chunk_decay`;
//   (gla_combine_kernel then walks a sequence's chunks in order: start_(c+1) = decay_c * start_c + local_c, puts each
//   chunk's start state where its local state was, and the last one into the sequence's state row)
//   mode OUTPUT   every chunk starts from its start state and writes its outputs.
// mode WHOLE is the recurrence in one pass, from and into the sequence's state row (decode steps, short prompts).
// Variants that other recurrences of this family need: `decay_per_head` (one decay per token and head, decay [T, H], for
// all its key channels), `key_gain` [T, H] (the key of a token is multiplied by it: an input gate), and `ones` (the last of
// the dv value columns is the constant 1 and the projection holds dv - 1 columns per head: that column of the state is
// then the decayed sum of the gated keys, and its output their product with the query: a normaliser). `bonus` [H, dk]
// (the time-mixing family): a token's output is formed from the state BEFORE the token plus u_c k_c v_j for the token
// itself, o_t = (S_(t-1) + diag(u) k_t v_t^T)^T q_t, and the state is updated afterwards.
constexpr int SCAN_WHOLE = 0, SCAN_LOCAL = 1, SCAN_OUTPUT = 2;

template <int KP, int VT, int KPT, int JT>
__global__ void __launch_bounds__(VT / JT * KP)
gla_scan_kernel(const float* __restrict__ proj, int ld, int q_off, int k_off, int v_off, const float* __restrict__ decay,
                float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ q_start,
                float* __restrict__ out, int H, int dk, int dv, float q_scale, int mode, int chunks, int chunk,
                float* __restrict__ chunk_state, float* __restrict__ chunk_decay, int decay_per_head,
                const float* __restrict__ key_gain, int ones, const float* __restrict__ bonus, int qk_group,
                const float* __restrict__ beta, int state_cols) {
    extern __shared__ float sm[];
    float* qs = sm;                         // [TB][dk]
    float* ks = qs + TB * dk;
    float* as = ks + TB * dk;
    float* vs = as + TB * dk;               // [TB][VT]
    lp_grid_release();
    lp_grid_wait();
    const int h = blockIdx.y, b = blockIdx.z / chunks, piece = blockIdx.z - b * chunks;
    // thread (column group jg, part): JT neighbouring value columns, so that a token's decays, keys and queries are
    // read from shared memory once for JT columns
    const int tid = threadIdx.x, part = tid % KP, jg = tid / KP;
    const int j0 = blockIdx.x * VT + jg * JT;
    int t0 = q_start[b], t1 = q_start[b + 1];
    if (mode != SCAN_WHOLE) {
        t0 += piece * chunk;
        t1 = min(t1, t0 + chunk);
        if (t0 >= t1) return;                             // this sequence has fewer chunks
    }
    // The delta rule in chunks side by side: a chunk's effect on the state that enters it is S -> P S + L with P a
    // [dk, dk] matrix (the product of the tokens' a (I - b k k^T)). Pass LOCAL therefore carries dk more columns per
    // head: they start as the identity, are fed the value 0, and end as P (column m of P in column dv + m);
    // `state_cols` = dv + dk is then how many columns a head has in `chunk_state` (else dv).
    const int cols = (beta && mode == SCAN_LOCAL) ? dv + dk : dv;
    float* S = mode == SCAN_WHOLE ? state + ((long long)slots[b] * H + h) * dv * dk
                                  : chunk_state + ((long long)blockIdx.z * H + h) * state_cols * dk;
    float s[KPT][JT], prod[KPT], ub[KPT];
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int c = part + KP * i;
        ub[i] = (bonus && c < dk) ? bonus[(long long)h * dk + c] : 0.f;
#pragma unroll
        for (int jj = 0; jj < JT; ++jj)
            s[i][jj] = (mode != SCAN_LOCAL && j0 + jj < dv && c < dk) ? S[(long long)(j0 + jj) * dk + c]
                       : ((beta && mode == SCAN_LOCAL && j0 + jj >= dv && c == j0 + jj - dv) ? 1.f : 0.f);
        prod[i] = 1.f;
    }
    for (int tb = t0; tb < t1; tb += TB) {
        const int nt = min(TB, t1 - tb);
        __syncthreads();
        for (int e = tid; e < nt * dk; e += blockDim.x) {
            const int i = e / dk, c = e - i * dk;
            const float* row = proj + (long long)(tb + i) * ld;
            qs[e] = row[q_off + (h / qk_group) * dk + c] * q_scale;
            ks[e] = row[k_off + (h / qk_group) * dk + c] * (key_gain ? key_gain[(long long)(tb + i) * H + h] : 1.0f);
            as[e] = decay_per_head ? decay[(long long)(tb + i) * H + h] : decay[((long long)(tb + i) * H + h) * dk + c];
        }
        for (int e = tid; e < nt * VT; e += blockDim.x) {
            const int i = e / VT, c = e - i * VT;
            const int col = blockIdx.x * VT + c;
            const int dvin = dv - ones;             // value columns that come from the projection
            vs[e] = col < dvin ? proj[(long long)(tb + i) * ld + v_off + h * dvin + col] : (col < dv ? 1.0f : 0.f);
        }
        __syncthreads();
        for (int i = 0; i < nt; ++i) {
            float v[JT], acc[JT];
#pragma unroll
            for (int jj = 0; jj < JT; ++jj) {
                v[jj] = vs[i * VT + jg * JT + jj];
                acc[jj] = 0.f;
            }
            const float* qi = qs + i * dk;
            const float* ki = ks + i * dk;
            const float* ai = as + i * dk;
            if (beta) {
                // the delta rule (one decay a per head): S <- a S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
                // Both read-outs are taken from the state before the token, S^T k and S^T q, in one pass of
                // shuffles: the decayed S^T k is a (S^T k), and o = a (S^T q) + u (k . q).
                float r1[JT], r2[JT], kq = 0.f;
#pragma unroll
                for (int jj = 0; jj < JT; ++jj) r1[jj] = r2[jj] = 0.f;
#pragma unroll
                for (int u = 0; u < KPT; ++u) {
                    const int c = part + KP * u;
                    if (c < dk) {
                        const float k = ki[c], q = qi[c];
                        kq = fmaf(k, q, kq);
#pragma unroll
                        for (int jj = 0; jj < JT; ++jj) {
                            r1[jj] = fmaf(s[u][jj], k, r1[jj]);
                            r2[jj] = fmaf(s[u][jj], q, r2[jj]);
                        }
                    }
                }
#pragma unroll
                for (int o = 1; o < KP; o <<= 1) {
                    kq += __shfl_xor_sync(0xffffffffu, kq, o);
#pragma unroll
                    for (int jj = 0; jj < JT; ++jj) {
                        r1[jj] += __shfl_xor_sync(0xffffffffu, r1[jj], o);
                        r2[jj] += __shfl_xor_sync(0xffffffffu, r2[jj], o);
                    }
                }
                const float a = ai[0];
                const float bt = beta[(long long)(tb + i) * H + h];
                float w[JT];
#pragma unroll
                for (int jj = 0; jj < JT; ++jj) {
                    w[jj] = bt * (v[jj] - a * r1[jj]);
                    acc[jj] = fmaf(w[jj], kq, a * r2[jj]);
                }
#pragma unroll
                for (int u = 0; u < KPT; ++u) {
                    const int c = part + KP * u;
                    if (c < dk) {
                        const float k = ki[c];
#pragma unroll
                        for (int jj = 0; jj < JT; ++jj) s[u][jj] = fmaf(a, s[u][jj], k * w[jj]);
                    }
                }
                if (mode != SCAN_LOCAL) {
#pragma unroll
                    for (int jj = 0; jj < JT; ++jj)
                        if (part == jj % KP && j0 + jj < dv) out[((long long)(tb + i) * H + h) * dv + j0 + jj] = acc[jj];
                }
                continue;
            }
#pragma unroll
            for (int u = 0; u < KPT; ++u) {
                const int c = part + KP * u;
                if (c < dk) {
                    const float a = ai[c], k = ki[c], q = qi[c];
                    if (mode == SCAN_LOCAL) prod[u] *= a;
                    if (bonus) {
#pragma unroll
                        for (int jj = 0; jj < JT; ++jj) {
                            const float kv = k * v[jj];
                            acc[jj] = fmaf(fmaf(ub[u], kv, s[u][jj]), q, acc[jj]);
                            s[u][jj] = fmaf(a, s[u][jj], kv);
                        }
                    } else {
#pragma unroll
                        for (int jj = 0; jj < JT; ++jj) {
                            s[u][jj] = fmaf(a, s[u][jj], k * v[jj]);
                            acc[jj] = fmaf(s[u][jj], q, acc[jj]);
                        }
                    }
                }
            }
            if (mode != SCAN_LOCAL) {
#pragma unroll
                for (int o = 1; o < KP; o <<= 1) {
#pragma unroll
                    for (int jj = 0; jj < JT; ++jj) acc[jj] += __shfl_xor_sync(0xffffffffu, acc[jj], o);
                }
#pragma unroll
                for (int jj = 0; jj < JT; ++jj)
                    if (part == jj % KP && j0 + jj < dv) out[((long long)(tb + i) * H + h) * dv + j0 + jj] = acc[jj];
            }
        }
    }
    if (mode == SCAN_OUTPUT) return;
#pragma unroll
    for (int i = 0; i < KPT; ++i) {
        const int c = part + KP * i;
#pragma unroll
        for (int jj = 0; jj < JT; ++jj)
            if (j0 + jj < cols && c < dk) S[(long long)(j0 + jj) * dk + c] = s[i][jj];
        if (mode == SCAN_LOCAL && !beta && blockIdx.x == 0 && jg == 0 && c < dk)
            chunk_decay[((long long)blockIdx.z * H + h) * dk + c] = prod[i];
    }
}

// One thread per state entry (sequence, head, value column, key channel) walks the sequence's chunks in order.
__global__ void __launch_bounds__(256)
gla_combine_kernel(float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ q_start,
                   float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int H, int dk, int dv,
                   int chunks, int chunk) {
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.y;
    const long long per = (long long)H * dv * dk;
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per) return;
    const int h = (int)(e / ((long long)dv * dk));
    const int c = (int)(e % dk);
    const int n = q_start[b + 1] - q_start[b];
    const int used = (n + chunk - 1) / chunk;
    float* row = state + (long long)slots[b] * per + e;
    float s = *row;
    for (int p = 0; p < used; ++p) {
        float* at = chunk_state + ((long long)b * chunks + p) * per + e;
        const float local = *at;
        *at = s;
        s = fmaf(chunk_decay[(((long long)b * chunks + p) * H + h) * dk + c], s, local);
    }
    *row = s;
}

// The delta rule's chunks in order: start_(p+1) = P_p start_p + L_p, column by column. One block per (value column,
// head, sequence) with a thread per key channel; the column of the current start state lies in shared memory. Each
// chunk's start state is put where its L was (columns 0 .. dv - 1 of the chunk's block), the last into the state row.
__global__ void __launch_bounds__(512)
delta_combine_kernel(float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ q_start,
                     float* __restrict__ chunk_state, int H, int dk, int dv, int chunks, int chunk) {
    __shared__ float col[512];
    lp_grid_release();
    lp_grid_wait();
    const int j = blockIdx.x, h = blockIdx.y, b = blockIdx.z, c = threadIdx.x;
    const int n = q_start[b + 1] - q_start[b];
    const int used = (n + chunk - 1) / chunk;
    const long long per = (long long)(dv + dk) * dk;
    float* row = state + (((long long)slots[b] * H + h) * dv + j) * dk;
    float mine = c < dk ? row[c] : 0.f;
    for (int p = 0; p < used; ++p) {
        if (c < dk) col[c] = mine;
        __syncthreads();
        float* blockp = chunk_state + (((long long)b * chunks + p) * H + h) * per;
        if (c < dk) {
            float acc = blockp[(long long)j * dk + c];                    // L_p[c][j]
            const float* P = blockp + (long long)dv * dk + c;             // P_p[c][m] lies at column dv + m, channel c
            int m = 0;
            for (; m + 32 <= dk; m += 32) {                               // 32 loads in flight: a block has few warps, and
                float pv[32];                                             // every chunk waits for the one before it
#pragma unroll
                for (int u = 0; u < 32; ++u) pv[u] = __ldcg(P + (long long)(m + u) * dk);
#pragma unroll
                for (int u = 0; u < 32; ++u) acc = fmaf(pv[u], col[m + u], acc);
            }
            for (; m + 8 <= dk; m += 8) {
                float pv[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) pv[u] = __ldcg(P + (long long)(m + u) * dk);
#pragma unroll
                for (int u = 0; u < 8; ++u) acc = fmaf(pv[u], col[m + u], acc);
            }
            for (; m < dk; ++m) acc = fmaf(__ldcg(P + (long long)m * dk), col[m], acc);
            blockp[(long long)j * dk + c] = mine;                         // the chunk's start state
            mine = acc;
        }
        __syncthreads();
    }
    if (c < dk) row[c] = mine;
}

// ---------------------------------------------------------------- exponential gates with a running maximum
// Per token and head, from the pre-activations zi, zf (float32 columns of the projection) and their biases:
//     i = cap * tanh((zi + bi) / cap)                       the logarithm of the input gate
//     f = logsigmoid(cap * tanh((zf + bf) / cap))           the logarithm of the forget gate
//     m_t = max(f + m_(t-1), i)                             the running maximum (the sequence's m starts at 0)
//     decay[t] = exp(f + m_(t-1) - m_t),  gain[t] = exp(i - m_t),  max_row[t] = m_t
// so that S_t = decay S_(t-1) + gain k v^T is the recurrence in a stabilised form (matrix memory of the xLSTM family).
// One block per sequence and head walks the sequence's new tokens 256 at a time. m is kept per slot and head in `mstate`.
__device__ __forceinline__ float lp_log_sigmoid(float v) { return -(fmaxf(-v, 0.f) + log1pf(expf(-fabsf(v)))); }

__global__ void __launch_bounds__(256)
exp_gates_kernel(const float* __restrict__ proj, int ld, int i_off, int f_off, const float* __restrict__ bias_i,
                 const float* __restrict__ bias_f, float cap, float* __restrict__ mstate, const int* __restrict__ slots,
                 const int* __restrict__ q_start, float* __restrict__ decay, float* __restrict__ gain,
                 float* __restrict__ max_row, int H) {
    __shared__ float warp_f[8], warp_i[8];
    __shared__ float ms[257];
    lp_grid_release();
    lp_grid_wait();
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    float* mp = mstate + (long long)slots[b] * H + h;
    float carry = *mp;
    const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
    // A token is the map m -> max(m + f, i); maps compose as (f1, i1) then (f2, i2) = (f1 + f2, max(i1 + f2, i2)), so
    // the maxima of 256 tokens at a time come from a scan over the block: within warps by shuffles, then over the warps.
    for (int base = t0; base < t1; base += 256) {
        const int t = base + tid;
        const bool valid = t < t1;
        float li = 0.f, lf = 0.f, F = 0.f, I = -INFINITY;          // the identity map for threads beyond the end
        if (valid) {
            const float zi = proj[(long long)t * ld + i_off + h] + bi;
            const float zf = proj[(long long)t * ld + f_off + h] + bf;
            li = cap > 0.f ? cap * tanhf(zi / cap) : zi;
            lf = lp_log_sigmoid(cap > 0.f ? cap * tanhf(zf / cap) : zf);
            F = lf;
            I = li;
        }
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float pf = __shfl_up_sync(0xffffffffu, F, o), pi = __shfl_up_sync(0xffffffffu, I, o);
            if (lane >= o) {
                I = fmaxf(pi + F, I);
                F = pf + F;
            }
        }
        if (lane == 31) { warp_f[warp] = F; warp_i[warp] = I; }
        __syncthreads();
        float af = 0.f, ai = -INFINITY;                            // the warps in front of this one
        for (int w = 0; w < warp; ++w) {
            ai = fmaxf(ai + warp_f[w], warp_i[w]);
            af += warp_f[w];
        }
        const float m = fmaxf(carry + (af + F), fmaxf(ai + F, I));
        ms[tid + 1] = m;
        if (tid == 0) ms[0] = carry;
        __syncthreads();
        if (valid) {
            const long long at = (long long)t * H + h;
            decay[at] = expf(lf + ms[tid] - m);
            gain[at] = expf(li - m);
            max_row[at] = m;
        }
        carry = ms[min(256, t1 - base)];
        __syncthreads();
    }
    if (tid == 0) *mp = carry;
}


// ---------------------------------------------------------------- token shift
// For the S maps of a time-mixing layer: out[s][t] = x_t + (x_(t-1) - x_t) * mu[s], where x_(t-1) of a sequence's first
// new token is the row kept for its slot in `last` (zeros at the sequence's start). One block per token; the block of a
// sequence's first new token alone reads that row, and, having read it, puts the sequence's last new token there.
template <typename TOut>
__global__ void __launch_bounds__(256)
token_shift_kernel(const float* __restrict__ x, float* __restrict__ last, const float* __restrict__ mu, const int* __restrict__ slots,
                   const int* __restrict__ q_start, const int* __restrict__ seq_ids, TOut* __restrict__ out, int T, int d, int S,
                   float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int t = blockIdx.x;
    const int b = seq_ids[t];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const bool first = t == t0;
    float* kept = last + (long long)slots[b] * d;
    const float* cur = x + (long long)t * d;
    const float* prev = first ? kept : cur - d;
    const float* newest = x + (long long)(t1 - 1) * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float c = cur[i], p = prev[i];
        if (first) kept[i] = newest[i];          // this thread has read kept[i]; no other block reads or writes it
        for (int s = 0; s < S; ++s)
            out[((long long)s * T + t) * d + i] = lp_from_float<TOut>(fmaf(p - c, mu[(long long)s * d + i], c));
    }
}

// The same, four neighbouring features per thread (rows of a multiple of four values): float4 loads, and for bfloat16
// blends one 8-byte store per blend.
template <typename TOut>
__global__ void __launch_bounds__(256)
token_shift_vec4_kernel(const float* __restrict__ x, float* __restrict__ last, const float* __restrict__ mu, const int* __restrict__ slots,
                        const int* __restrict__ q_start, const int* __restrict__ seq_ids, TOut* __restrict__ out, int T, int d, int S,
                        float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int t = blockIdx.x;
    const int b = seq_ids[t];
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const bool first = t == t0;
    float* kept = last + (long long)slots[b] * d;
    const float* cur = x + (long long)t * d;
    const float* prev = first ? kept : cur - d;
    const float* newest = x + (long long)(t1 - 1) * d;
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        const float4 c = *reinterpret_cast<const float4*>(cur + i);
        const float4 p = *reinterpret_cast<const float4*>(prev + i);
        if (first) *reinterpret_cast<float4*>(kept + i) = *reinterpret_cast<const float4*>(newest + i);
        for (int s = 0; s < S; ++s) {
            const float4 m = *reinterpret_cast<const float4*>(mu + (long long)s * d + i);
            const float v0 = fmaf(p.x - c.x, m.x, c.x), v1 = fmaf(p.y - c.y, m.y, c.y);
            const float v2 = fmaf(p.z - c.z, m.z, c.z), v3 = fmaf(p.w - c.w, m.w, c.w);
            TOut* at = out + ((long long)s * T + t) * d + i;
            if constexpr (sizeof(TOut) == 4) {
                *reinterpret_cast<float4*>(at) = make_float4(v0, v1, v2, v3);
            } else {
                uint2 packed;
                *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v0, v1);
                *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v2, v3);
                *reinterpret_cast<uint2*>(at) = packed;
            }
        }
    }
}

// ---------------------------------------------------------------- finish
// out[t, h * dv + j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * gain[j] * silu(gate[t, h * dv + j]); a warp per (t, h).
// Variants: rows of o that are `xs` apart (xs > dv: further columns follow a head's values), a gain per head
// (`gain_per_head`: gain [H * dv]), a sigmoid instead of the silu (`gate_sigmoid`), and `max_row` [T, H] (see the kernel).
template <typename TOut>
__global__ void __launch_bounds__(256)
gla_finish_kernel(const float* __restrict__ o, const float* __restrict__ gain, float eps, const float* __restrict__ gate,
                  int ldg, TOut* __restrict__ out, int T, int H, int dv, float* __restrict__ zero, long long zero_count,
                  int xs, int gain_per_head, int gate_sigmoid, const float* __restrict__ max_row) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= (long long)T * H) return;
    const long long t = row / H;
    const int h = (int)(row - t * H);
    const float* x = o + row * xs;
    // with a normaliser column (x[dv]) and the row's running maximum m: x / (max(|x[dv]|, exp(-m)) + 1e-6) first
    const float pre = max_row ? 1.0f / (fmaxf(fabsf(x[dv]), expf(-max_row[row])) + 1e-6f) : 1.0f;
    float ss = 0.f;
    for (int j = lane; j < dv; j += 32) {
        const float v = x[j] * pre;
        ss += v * v;
    }
    ss = lp_warp_sum(ss);
    const float factor = pre / sqrtf(ss / (float)dv + eps);
    const float* g = gate ? gate + t * ldg + (long long)h * dv : nullptr;
    const float* gn = gain_per_head ? gain + (long long)h * dv : gain;
    for (int j = lane; j < dv; j += 32) {
        float v = x[j] * factor * gn[j];
        if (g) v *= gate_sigmoid ? 1.0f / (1.0f + expf(-g[j])) : g[j] / (1.0f + expf(-g[j]));
        out[row * dv + j] = lp_from_float<TOut>(v);
    }
}


// ---------------------------------------------------------------- short causal convolution with a carried tail
// out[t, c] = act(bias[c] + sum_j taps[c, j] * in[t - (K - 1) + j, c]), K taps per channel, the last one on the token
// itself; inputs before a sequence's first token are zero, inputs before the step's first token come from the K - 1
// rows kept for the sequence's slot in `tail` [slots, K - 1, C] (oldest first), which afterwards holds the step's
// last K - 1 inputs. grid (channels / 128, chunks of CONV_CHUNK tokens, sequences): a thread owns one channel of one
// chunk and walks its tokens in order with the K - 1 inputs before them in registers. Only a sequence's first chunk
// reads the tail (CONV_CHUNK >= K - 1), and the same thread, having read it, writes the new one.
constexpr int CONV_CHUNK = 32;
constexpr int CONV_MAX_TAPS = 8;

template <typename TW>
__global__ void __launch_bounds__(128)
short_conv_kernel(const float* __restrict__ in, int ldi, const TW* __restrict__ taps, const float* __restrict__ bias,
                  float* __restrict__ tail, const int* __restrict__ slots, const int* __restrict__ q_start,
                  float* __restrict__ out, int ldo, int C, int K, int silu) {
    lp_grid_release();
    lp_grid_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.z;
    const int t0 = q_start[b], t1 = q_start[b + 1];
    const int begin = t0 + blockIdx.y * CONV_CHUNK;
    if (c >= C || begin >= t1) return;
    const int end = min(t1, begin + CONV_CHUNK);
    // taps and the inputs before the token, both aligned at their ends: w[7] multiplies the token itself, w[6] and
    // hist[6] belong to the token before it, and so on; taps beyond K are zero, so all seven places always take part
    float w[CONV_MAX_TAPS], hist[CONV_MAX_TAPS - 1];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        const int tap = j - (CONV_MAX_TAPS - K);
        w[j] = tap >= 0 ? lp_to_float(taps[(long long)c * K + tap]) : 0.f;
    }
    float* keep = tail + (long long)slots[b] * (K - 1) * C + c;
#pragma unroll
    for (int i = 0; i < CONV_MAX_TAPS - 1; ++i) {               // hist[6 - i]: the input i + 1 tokens before `begin`
        float v = 0.f;
        if (i < K - 1) {
            const int src = begin - 1 - i;
            v = src >= t0 ? in[(long long)src * ldi + c] : keep[(long long)(K - 1 + src - t0) * C];
        }
        hist[CONV_MAX_TAPS - 2 - i] = v;
    }
    if (begin == t0) {
        // the step's last K - 1 inputs become the tail: new tokens where there are enough, else older rows move up
        // (row j takes row j + n, which is still unwritten when row j is)
        const int n = t1 - t0;
        for (int j = 0; j < K - 1; ++j) {
            const int src = t1 - (K - 1) + j;                  // token index of the j-th row of the new tail
            keep[(long long)j * C] = src >= t0 ? in[(long long)src * ldi + c] : keep[(long long)(j + n) * C];
        }
    }
    const float bv = bias ? bias[c] : 0.f;
    for (int t = begin; t < end; ++t) {
        const float x = in[(long long)t * ldi + c];
        float acc = bv;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) acc = fmaf(w[j], hist[j], acc);
        acc = fmaf(w[CONV_MAX_TAPS - 1], x, acc);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 2; ++j) hist[j] = hist[j + 1];
        hist[CONV_MAX_TAPS - 2] = x;
        out[(long long)t * ldo + c] = silu ? acc / (1.0f + expf(-acc)) : acc;
    }
}

// ---------------------------------------------------------------- step sizes, decays and write strengths of a recurrence
// Per token and head, from float32 columns of a projection: dt = softplus(z + dt_bias[h]) (no clamp),
// decay = exp(-exp(a_log[h]) * dt), and, where a second column zb is given, strength = sigmoid(zb).
__global__ void __launch_bounds__(256)
decay_gates_kernel(const float* __restrict__ proj, int ld, int z_off, int b_off, const float* __restrict__ dt_bias,
                   const float* __restrict__ a_log, float* __restrict__ decay, float* __restrict__ dt_out,
                   float* __restrict__ strength, int T, int H) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * H;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / H;
        const int h = (int)(i - t * H);
        const float z = proj[t * ld + z_off + h] + (dt_bias ? dt_bias[h] : 0.f);
        const float dt = z > 20.f ? z : log1pf(expf(z));
        decay[i] = expf(-expf(a_log[h]) * dt);
        if (dt_out) dt_out[i] = dt;
        if (strength) strength[i] = 1.0f / (1.0f + expf(-proj[t * ld + b_off + h]));
    }
}

// ---------------------------------------------------------------- heads made unit vectors
// x[t, off + h * dim + i] <- x / sqrt(sum_i x^2 + eps), in place, float32; the first `scaled` heads also times `scale`
// (queries in front of keys). A warp per (token, head).
__global__ void __launch_bounds__(128)
head_unit_norm_kernel(float* __restrict__ x, int ld, int off, int heads, int dim, float eps, float scale, int scaled, int T) {
    lp_grid_release();
    lp_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 4 + warp;
    if (row >= (long long)T * heads) return;
    const long long t = row / heads;
    const int h = (int)(row - t * heads);
    float* v = x + t * ld + off + (long long)h * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) ss = fmaf(v[i], v[i], ss);
    ss = lp_warp_sum(ss);
    const float f = (h < scaled ? scale : 1.0f) / sqrtf(ss + eps);
    for (int i = lane; i < dim; i += 32) v[i] *= f;
}

// ---------------------------------------------------------------- skip, gate, then a norm in equal parts
// y[t, h * P + i] = (raw[t, h * P + i] + skip[h] * x[t, h * P + i]) * silu(z[t, h * P + i]); the row of H * P values is
// then cut into `parts` equal parts, each divided by its own root mean square (eps inside the root) and multiplied by
// the gain. One block per (token, part). The gate comes before the norm.
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_part_norm_kernel(const float* __restrict__ raw, const float* __restrict__ x, int ldx, const float* __restrict__ skip,
                       const float* __restrict__ z, int ldz, const float* __restrict__ gain, float eps, TOut* __restrict__ out,
                       int P, int width, int part_width, float* __restrict__ zero, long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long t = blockIdx.x;
    const int base = blockIdx.y * part_width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < part_width; i += blockDim.x) {
        const int col = base + i;
        const float g = z[t * ldz + col];
        float y = raw[t * width + col];
        if (skip) y = fmaf(skip[col / P], x[t * ldx + col], y);
        y *= g / (1.0f + expf(-g));
        ss = fmaf(y, y, ss);
    }
    ss = lp_block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)part_width + eps);
    for (int i = threadIdx.x; i < part_width; i += blockDim.x) {
        const int col = base + i;
        const float g = z[t * ldz + col];
        float y = raw[t * width + col];
        if (skip) y = fmaf(skip[col / P], x[t * ldx + col], y);
        y *= g / (1.0f + expf(-g));
        out[t * width + col] = lp_from_float<TOut>(y * f * gain[col]);
    }
}

}  // namespace

// form 0: sigmoid(z)^(1 / tau) with z = a2 low + bias; form 1: exp(-exp(z)) with z = a2 tanh(low) + bias (tau unused).
extern "C" int lp_gla_decay(const float* low, int ldl, const void* a2, int w_dtype, const float* bias, float* out,
                            int T, int C, int R, float tau, int form, cudaStream_t stream) {
    if (T <= 0 || C <= 0) return 0;
    if (R <= 0 || ldl < R) LP_REFUSE("gla_decay: a factor of %d values in rows of %d", R, ldl);
    if (form < 0 || form > 1) LP_REFUSE("gla_decay: form %d", form);
    if (form == 1) tau = 1.0f;
    if (!(tau > 0.f)) LP_REFUSE("gla_decay: temperature %g", (double)tau);
    const long long n = (long long)T * C;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (w_dtype == LP_F32)
        lp_launch(gla_decay_kernel<float>, (unsigned)blocks, 256, 0, stream, low, ldl, (const float*)a2, bias, out, T, C, R, 1.0f / tau, form);
    else if (w_dtype == LP_BF16)
        lp_launch(gla_decay_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, low, ldl, (const __nv_bfloat16*)a2, bias, out, T, C, R, 1.0f / tau, form);
    else LP_REFUSE("gla_decay: weight dtype code %d", w_dtype);
    return lp_check_launch("gla_decay");
}

// proj: float32 [T, ld] with queries at q_off ([H, dk]), keys at k_off ([H, dk]), values at v_off ([H, dv]);
// decay: float32 [T, H * dk]; state: float32 [slots, H, dv, dk]; out: float32 [T, H, dv].
// chunks > 1 (with chunk tokens each, chunk_state float32 [B, chunks, H, dv, dk], chunk_decay float32 [B, chunks, H, dk]):
// the chunks of a sequence run side by side in three launches; every sequence needs at most `chunks` chunks.
extern "C" int lp_gla_scan(const float* proj, int ld, int q_off, int k_off, int v_off, const float* decay, float* state,
                           const int* slots, const int* q_start, float* out, int B, int H, int dk, int dv,
                           float q_scale, int chunks, int chunk, float* chunk_state, float* chunk_decay,
                           int decay_per_head, const float* key_gain, int ones, const float* bonus, int qk_heads,
                           const float* beta, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (chunks < 1) chunks = 1;
    // queries and keys may have fewer heads than the values: head h then reads query / key head h / (H / qk_heads)
    if (qk_heads <= 0) qk_heads = H;
    if (H % qk_heads) LP_REFUSE("gla_scan: %d heads over %d query / key heads", H, qk_heads);
    const int qk_group = H / qk_heads;
    const int state_cols = (beta && chunks > 1) ? dv + dk : dv;      // columns of a head in `chunk_state`
    if (beta && (!decay_per_head || bonus || ones)) LP_REFUSE("gla_scan: the delta rule takes one decay per head and no bonus");
    ones = ones ? 1 : 0;
    if (dv - ones <= 0) LP_REFUSE("gla_scan: %d value columns, %d of them constant", dv, ones);
    if (chunks > 1 && (chunk <= 0 || !chunk_state || (!chunk_decay && !beta))) LP_REFUSE("gla_scan: %d chunks without their buffers", chunks);
    if ((long long)B * chunks > 65535) LP_REFUSE("gla_scan: %d sequences in %d chunks exceed the grid", B, chunks);
    if (H <= 0 || H > 65535 || B > 65535 || dk <= 0 || dv <= 0) LP_REFUSE("gla_scan: %d sequences, %d heads of %d x %d", B, H, dk, dv);
    if (dk > 512) LP_REFUSE("gla_scan: %d key channels per head (supported: up to 512)", dk);
    if (q_off < 0 || k_off < 0 || v_off < 0 || q_off + qk_heads * dk > ld || k_off + qk_heads * dk > ld || v_off + H * (dv - (ones ? 1 : 0)) > ld)
        LP_REFUSE("gla_scan: slices at %d, %d, %d do not fit rows of %d", q_off, k_off, v_off, ld);
#define LP_LAUNCH_SCAN(KP_, VT_, N, JT_)                                                                                 \
    do {                                                                                                              \
        dim3 grid((dv + VT_ - 1) / VT_, H, B * chunks);                                                               \
        const size_t smem = ((size_t)3 * TB * dk + (size_t)TB * VT_) * sizeof(float);                                 \
        if (smem > 48 * 1024) {                                                                                       \
            cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel<KP_, VT_, N, JT_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) LP_REFUSE("gla_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e)); \
        }                                                                                                             \
        if (chunks == 1) {                                                                                            \
            lp_launch(gla_scan_kernel<KP_, VT_, N, JT_>, grid, VT_ / JT_ * KP_, smem, stream, proj, ld, q_off, k_off, v_off,     \
                      decay, state, slots, q_start, out, H, dk, dv, q_scale, SCAN_WHOLE, 1, 0, (float*)nullptr,       \
                      (float*)nullptr, decay_per_head, key_gain, ones, bonus, qk_group, beta, state_cols);                                                                               \
        } else {                                                                                                      \
            dim3 grid_local((state_cols + VT_ - 1) / VT_, H, B * chunks);                                             \
            lp_launch(gla_scan_kernel<KP_, VT_, N, JT_>, grid_local, VT_ / JT_ * KP_, smem, stream, proj, ld, q_off, k_off, v_off,     \
                      decay, state, slots, q_start, out, H, dk, dv, q_scale, SCAN_LOCAL, chunks, chunk, chunk_state,  \
                      chunk_decay, decay_per_head, key_gain, ones, bonus, qk_group, beta, state_cols);                                                                                   \
            const long long per = (long long)H * dv * dk;                                                             \
            if (beta)                                                                                                 \
                lp_launch(delta_combine_kernel, dim3(dv, H, B), (dk + 31) / 32 * 32, 0, stream, state, slots, q_start, \
                          chunk_state, H, dk, dv, chunks, chunk);                                                     \
            else                                                                                                      \
                lp_launch(gla_combine_kernel, dim3((unsigned)((per + 255) / 256), B), 256, 0, stream, state, slots,   \
                          q_start, chunk_state, (const float*)chunk_decay, H, dk, dv, chunks, chunk);                 \
            lp_launch(gla_scan_kernel<KP_, VT_, N, JT_>, grid, VT_ / JT_ * KP_, smem, stream, proj, ld, q_off, k_off, v_off,     \
                      decay, state, slots, q_start, out, H, dk, dv, q_scale, SCAN_OUTPUT, chunks, chunk, chunk_state, \
                      chunk_decay, decay_per_head, key_gain, ones, bonus, qk_group, beta, state_cols);                                                                                   \
        }                                                                                                             \
    } while (0)
    // few key channels: 4 threads per column, 64 columns per CTA; from 32 channels on: 16 threads per column, 16 columns
    // (threads per column, columns per CTA, channels per thread, columns per thread): 256 threads in every form
    if (dk <= 8) LP_LAUNCH_SCAN(4, 64, 2, 1);
    else if (dk <= 16) LP_LAUNCH_SCAN(4, 64, 4, 1);
    else if (dk < 32) LP_LAUNCH_SCAN(4, 64, 8, 1);
    else if (dk <= 64) LP_LAUNCH_SCAN(16, 64, 4, 4);
    else if (dk <= 128) LP_LAUNCH_SCAN(16, 64, 8, 4);
    else if (dk <= 256) LP_LAUNCH_SCAN(16, 32, 16, 2);
    else LP_LAUNCH_SCAN(16, 16, 32, 1);
#undef LP_LAUNCH_SCAN
    return lp_check_launch("gla_scan");
}

extern "C" int lp_gla_finish(const float* o, const float* gain, float eps, const float* gate, int ldg, void* out,
                             int out_dtype, int T, int H, int dv, float* zero, long long zero_count, int xs,
                             int gain_per_head, int gate_sigmoid, const float* max_row, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || dv <= 0) LP_REFUSE("gla_finish: %d heads of %d", H, dv);
    if (xs <= 0) xs = dv;
    if (xs < dv || (max_row && xs < dv + 1)) LP_REFUSE("gla_finish: rows %d apart for %d values", xs, dv);
    const long long rows = (long long)T * H;
    const unsigned blocks = (unsigned)((rows + 7) / 8);
    if (out_dtype == LP_F32) lp_launch(gla_finish_kernel<float>, blocks, 256, 0, stream, o, gain, eps, gate, ldg, (float*)out, T, H, dv, zero, zero_count, xs, gain_per_head, gate_sigmoid, max_row);
    else if (out_dtype == LP_BF16)
        lp_launch(gla_finish_kernel<__nv_bfloat16>, blocks, 256, 0, stream, o, gain, eps, gate, ldg, (__nv_bfloat16*)out, T, H, dv, zero, zero_count, xs, gain_per_head, gate_sigmoid, max_row);
    else LP_REFUSE("gla_finish: output dtype code %d", out_dtype);
    return lp_check_launch("gla_finish");
}

// proj: float32 [T, ld] with the input gate's pre-activations at i_off and the forget gate's at f_off (H each);
// bias_i, bias_f: float32 [H] or null; cap <= 0: no cap. mstate: float32 [slots, H]; decay, gain, max_row: float32 [T, H].
extern "C" int lp_exp_gates(const float* proj, int ld, int i_off, int f_off, const float* bias_i, const float* bias_f,
                            float cap, float* mstate, const int* slots, const int* q_start, float* decay, float* gain,
                            float* max_row, int B, int H, cudaStream_t stream) {
    if (B <= 0) return 0;
    if (H <= 0 || i_off < 0 || f_off < 0 || i_off + H > ld || f_off + H > ld)
        LP_REFUSE("exp_gates: %d heads at %d and %d in rows of %d", H, i_off, f_off, ld);
    if (H > 65535) LP_REFUSE("exp_gates: %d heads exceed the grid", H);
    lp_launch(exp_gates_kernel, dim3(B, H), 256, 0, stream, proj, ld, i_off, f_off, bias_i, bias_f, cap, mstate, slots, q_start,
              decay, gain, max_row, H);
    return lp_check_launch("exp_gates");
}

// x: float32 [T, d]; last: float32 [slots, d]; mu: float32 [S, d]; out: [S, T, d] float32 or bfloat16.
extern "C" int lp_token_shift(const float* x, float* last, const float* mu, const int* slots, const int* q_start,
                              const int* seq_ids, void* out, int out_dtype, int T, int d, int S, float* zero, long long zero_count,
                              cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0 || S <= 0) LP_REFUSE("token_shift: rows of %d values, %d blends", d, S);
    const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(last) | reinterpret_cast<uintptr_t>(mu) |
                           reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (d % 4 == 0 && aligned && (out_dtype == LP_F32 || out_dtype == LP_BF16)) {
        const int threads = d >= 1024 ? 256 : d >= 512 ? 128 : 64;
        if (out_dtype == LP_F32) lp_launch(token_shift_vec4_kernel<float>, T, threads, 0, stream, x, last, mu, slots, q_start, seq_ids, (float*)out, T, d, S, zero, zero_count);
        else lp_launch(token_shift_vec4_kernel<__nv_bfloat16>, T, threads, 0, stream, x, last, mu, slots, q_start, seq_ids, (__nv_bfloat16*)out, T, d, S, zero, zero_count);
        return lp_check_launch("token_shift");
    }
    if (out_dtype == LP_F32) lp_launch(token_shift_kernel<float>, T, 256, 0, stream, x, last, mu, slots, q_start, seq_ids, (float*)out, T, d, S, zero, zero_count);
    else if (out_dtype == LP_BF16) lp_launch(token_shift_kernel<__nv_bfloat16>, T, 256, 0, stream, x, last, mu, slots, q_start, seq_ids, (__nv_bfloat16*)out, T, d, S, zero, zero_count);
    else LP_REFUSE("token_shift: output dtype code %d", out_dtype);
    return lp_check_launch("token_shift");
}

// in: float32 [T, ldi] (C channels from the given pointer); taps: [C, K]; bias: float32 [C] or null; tail: float32
// [slots, K - 1, C]; out: float32 [T, ldo]. max_new: most new tokens of a sequence of the step.
extern "C" int lp_short_conv(const float* in, int ldi, const void* taps, int w_dtype, const float* bias, float* tail,
                             const int* slots, const int* q_start, float* out, int ldo, int B, int max_new, int C, int K,
                             int silu, cudaStream_t stream) {
    if (B <= 0 || max_new <= 0 || C <= 0) return 0;
    if (K < 1 || K > CONV_MAX_TAPS) LP_REFUSE("short_conv: %d taps (supported: 1..%d)", K, CONV_MAX_TAPS);
    if (ldi < C || ldo < C) LP_REFUSE("short_conv: rows of %d and %d values for %d channels", ldi, ldo, C);
    const int chunks = (max_new + CONV_CHUNK - 1) / CONV_CHUNK;
    if (chunks > 65535 || B > 65535) LP_REFUSE("short_conv: %d chunks of tokens, %d sequences exceed the grid", chunks, B);
    dim3 grid((C + 127) / 128, chunks, B);
    if (w_dtype == LP_F32) lp_launch(short_conv_kernel<float>, grid, 128, 0, stream, in, ldi, (const float*)taps, bias, tail, slots, q_start, out, ldo, C, K, silu);
    else if (w_dtype == LP_BF16) lp_launch(short_conv_kernel<__nv_bfloat16>, grid, 128, 0, stream, in, ldi, (const __nv_bfloat16*)taps, bias, tail, slots, q_start, out, ldo, C, K, silu);
    else LP_REFUSE("short_conv: dtype code %d of the taps", w_dtype);
    return lp_check_launch("short_conv");
}

// proj: float32 [T, ld]; z_off: column of the H step-size pre-activations; b_off: column of the H write-strength
// pre-activations (used only with `strength`); decay, dt_out (optional), strength (optional): float32 [T, H].
extern "C" int lp_decay_gates(const float* proj, int ld, int z_off, int b_off, const float* dt_bias, const float* a_log,
                              float* decay, float* dt_out, float* strength, int T, int H, cudaStream_t stream) {
    if (T <= 0 || H <= 0) return 0;
    if (z_off < 0 || z_off + H > ld || (strength && (b_off < 0 || b_off + H > ld))) LP_REFUSE("decay_gates: columns at %d / %d of rows of %d", z_off, b_off, ld);
    long long blocks = ((long long)T * H + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    lp_launch(decay_gates_kernel, (unsigned)blocks, 256, 0, stream, proj, ld, z_off, b_off, dt_bias, a_log, decay, dt_out, strength, T, H);
    return lp_check_launch("decay_gates");
}

extern "C" int lp_head_unit_norm(float* x, int ld, int off, int heads, int dim, float eps, float scale, int scaled, int T,
                                 cudaStream_t stream) {
    if (T <= 0 || heads <= 0 || dim <= 0) return 0;
    if (off < 0 || off + heads * dim > ld) LP_REFUSE("head_unit_norm: %d heads of %d at column %d of rows of %d", heads, dim, off, ld);
    const long long rows = (long long)T * heads;
    lp_launch(head_unit_norm_kernel, (unsigned)((rows + 3) / 4), 128, 0, stream, x, ld, off, heads, dim, eps, scale, scaled, T);
    return lp_check_launch("head_unit_norm");
}

// raw: float32 [T, H * P]; x: float32 [T, ldx] (the values, for the skip) with skip float32 [H], both or neither;
// z: float32 [T, ldz] gate pre-activations; gain: float32 [H * P]; out: [T, H * P]; parts: equal parts of a row.
extern "C" int lp_gated_part_norm(const float* raw, const float* x, int ldx, const float* skip, const float* z, int ldz,
                                  const float* gain, float eps, void* out, int dtype, int T, int H, int P, int parts,
                                  float* zero, long long zero_count, cudaStream_t stream) {
    if (T <= 0) return 0;
    const int width = H * P;
    if (H <= 0 || P <= 0 || parts <= 0 || width % parts || parts > 65535) LP_REFUSE("gated_part_norm: %d heads of %d in %d parts", H, P, parts);
    if ((skip != nullptr) != (x != nullptr)) LP_REFUSE("gated_part_norm: a skip comes with the values it multiplies");
    if (ldz < width || (x && ldx < width)) LP_REFUSE("gated_part_norm: rows of %d / %d values for %d columns", ldz, ldx, width);
    dim3 grid(T, parts);
    if (dtype == LP_F32) lp_launch(gated_part_norm_kernel<float>, grid, 256, 0, stream, raw, x, ldx, skip, z, ldz, gain, eps, (float*)out, P, width, width / parts, zero, zero_count);
    else if (dtype == LP_BF16) lp_launch(gated_part_norm_kernel<__nv_bfloat16>, grid, 256, 0, stream, raw, x, ldx, skip, z, ldz, gain, eps, (__nv_bfloat16*)out, P, width, width / parts, zero, zero_count);
    else LP_REFUSE("gated_part_norm: dtype code %d", dtype);
    return lp_check_launch("gated_part_norm");
}
