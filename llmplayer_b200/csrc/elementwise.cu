// Small memory-bound kernels of the step: embedding rows, RMS norm, and the
// rotation of queries and keys together with the write of keys and values into
// the paged cache. All arithmetic is float32; only loads and stores convert.
//
// Counterparts in the reference (src/main/resources/kernels/cuda/): rmsnorm.cu:6-46,
// rope.cu:11-52, attention.cu:114-128 (kv_cache_update); the embedding row is
// gathered on the host there (inference/InferenceEngine.java:199-201).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embed_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int d, float scale) {
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const long long row = tokens[t];
    const TW* src = table + row * d;
    float* dst = out + (long long)t * d;
    // a scale of one leaves the row as stored (no multiplication, the same bits)
    if (scale == 1.0f) {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = lp_to_float(src[i]);
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = lp_to_float(src[i]) * scale;
    }
}

extern "C" int lp_embed(const void* table, int table_dtype, const int* tokens, float* out, int T, int d,
                        float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (d <= 0) LP_REFUSE("embed: width %d", d);
    const int threads = d >= 1024 ? 256 : 128;
    // the embedding opens a step: it is launched without the early start (see lp_launch_first)
    if (table_dtype == LP_F32)
        lp_launch_first(embed_kernel<float>, T, threads, 0, stream, (const float*)table, tokens, out, d, scale);
    else if (table_dtype == LP_BF16)
        lp_launch_first(embed_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)table, tokens, out, d, scale);
    else
        LP_REFUSE("embed: table dtype code %d", table_dtype);
    return lp_check_launch("embed");
}

// ---------------------------------------------------------------- RMS norm
// out[r, i] = x[row(r), i] * (1 / sqrt(sum_i x^2 / d + eps)) * w[i]; one block per row.
// When `add` is given, x[row] += add[row] first (in float32) and the sum is stored back:
// the residual sum and the norm that follows it in one pass. The row is read once and kept
// in registers (up to PER * 256 values; wider rows take the two-pass kernel below).
// `zero` (optional): a float32 buffer that the blocks clear on the side, for the product that
// follows the norm and sums its partial results with atomics.
constexpr int NORM_THREADS = 256;
constexpr int NORM_PER = 16;


template <typename TOut, typename TAdd>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_kernel(float* __restrict__ x, const TAdd* __restrict__ add, const int* __restrict__ rows,
               const float* __restrict__ w, TOut* __restrict__ out, int d, float eps, float* __restrict__ zero,
               long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float* xr = x + src * d;
    float v[NORM_PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        v[k] = 0.f;
        if (i < d) {
            float t = xr[i];
            if (add) { t += lp_to_float(add[src * d + i]); xr[i] = t; }
            v[k] = t;
            ss += t * t;
        }
    }
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TOut* o = out + (long long)r * d;
#pragma unroll
    for (int k = 0; k < NORM_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < d) o[i] = lp_from_float<TOut>(v[k] * scale * w[i]);
    }
}

// The same for rows of a multiple of 4 values without a residual add: four values per load and store.
constexpr int NORM_VEC_PER = 4;          // float4 per thread: rows up to 256 * 4 * 4 = 4096 values
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_vec4_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                    TOut* __restrict__ out, int d, float eps, float* __restrict__ zero, long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    const float4* xr = reinterpret_cast<const float4*>(x + src * d);
    const int quads = d >> 2;
    float4 v[NORM_VEC_PER];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < quads) v[k] = xr[i];
    }
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    const float4* wq = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int k = 0; k < NORM_VEC_PER; ++k) {
        const int i = threadIdx.x + k * NORM_THREADS;
        if (i < quads) {
            const float4 g = wq[i];
            const float a = v[k].x * scale * g.x, b = v[k].y * scale * g.y, c = v[k].z * scale * g.z, e = v[k].w * scale * g.w;
            if (sizeof(TOut) == 2) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, e);
                uint2 packed;
                packed.x = *reinterpret_cast<uint32_t*>(&lo);
                packed.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(out + (long long)r * d)[i] = packed;
            } else {
                reinterpret_cast<float4*>(out + (long long)r * d)[i] = make_float4(a, b, c, e);
            }
        }
    }
}

template <typename TOut, typename TAdd>
__global__ void rmsnorm_wide_kernel(float* __restrict__ x, const TAdd* __restrict__ add,
                                    const int* __restrict__ rows, const float* __restrict__ w,
                                    TOut* __restrict__ out, int d, float eps, float* __restrict__ zero,
                                    long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    float* xr = x + src * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float t = xr[i];
        if (add) { t += lp_to_float(add[src * d + i]); xr[i] = t; }
        ss += t * t;
    }
    clear_on_the_side(zero, zero_count);
    ss = lp_block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)d + eps);
    TOut* o = out + (long long)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = lp_from_float<TOut>(xr[i] * scale * w[i]);
}

extern "C" int lp_rmsnorm(float* x, const void* add, int add_dtype, const int* rows, const float* w, void* out,
                          int out_dtype, int R, int d, float eps, float* zero, long long zero_count,
                          cudaStream_t stream) {
    if (R <= 0) return 0;
    if (d <= 0) LP_REFUSE("rmsnorm: width %d", d);
    if (add && rows) LP_REFUSE("rmsnorm: a fused residual add cannot be combined with a row selection");
    const bool wide = d > NORM_THREADS * NORM_PER;
    if (!add && d % 4 == 0 && d <= NORM_THREADS * 4 * NORM_VEC_PER &&
        ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out) & 15) == 0)) {
        if (out_dtype == LP_BF16)
            lp_launch(rmsnorm_vec4_kernel<__nv_bfloat16>, R, NORM_THREADS, 0, stream, (const float*)x, rows, w,
                      (__nv_bfloat16*)out, d, eps, zero, zero_count);
        else if (out_dtype == LP_F32)
            lp_launch(rmsnorm_vec4_kernel<float>, R, NORM_THREADS, 0, stream, (const float*)x, rows, w, (float*)out, d,
                      eps, zero, zero_count);
        else LP_REFUSE("rmsnorm: dtype code out=%d", out_dtype);
        return lp_check_launch("rmsnorm");
    }
#define LP_LAUNCH_NORM(TOUT, TADD)                                                                              \
    do {                                                                                                        \
        if (wide)                                                                                               \
            lp_launch(rmsnorm_wide_kernel<TOUT, TADD>, R, 512, 0, stream, x, (const TADD*)add, rows, w,          \
                      (TOUT*)out, d, eps, zero, zero_count);                                                    \
        else                                                                                                    \
            lp_launch(rmsnorm_kernel<TOUT, TADD>, R, NORM_THREADS, 0, stream, x, (const TADD*)add, rows, w,      \
                      (TOUT*)out, d, eps, zero, zero_count);                                                    \
    } while (0)
    if (out_dtype == LP_F32 && add_dtype == LP_F32) LP_LAUNCH_NORM(float, float);
    else if (out_dtype == LP_F32 && add_dtype == LP_BF16) LP_LAUNCH_NORM(float, __nv_bfloat16);
    else if (out_dtype == LP_BF16 && add_dtype == LP_F32) LP_LAUNCH_NORM(__nv_bfloat16, float);
    else if (out_dtype == LP_BF16 && add_dtype == LP_BF16) LP_LAUNCH_NORM(__nv_bfloat16, __nv_bfloat16);
    else LP_REFUSE("rmsnorm: dtype codes out=%d add=%d", out_dtype, add_dtype);
#undef LP_LAUNCH_NORM
    return lp_check_launch("rmsnorm");
}

// ---------------------------------------------------------------- rotation + cache write
// One block per token of the fused projection output
//   qkv[t] = [ H query heads | G key heads | G value heads ] x head_dim   (float32).
// Queries and keys: the first `rd` features of a head are rotated by
// angle = float(position) * inv_freq[pair] (cosine and sine are formed once per token and
// shared by all its heads); the rest pass through. Queries go to q_out[t, h, :]; keys and
// values go to the page of the token's sequence that holds its position:
//   pages[page][0|1][g][position % page_size][:].
template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rope_cache_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ inv_freq,
                  const int* __restrict__ positions, const int* __restrict__ seq_ids,
                  const int* __restrict__ page_table, int pt_stride, TQ* __restrict__ q_out,
                  TKV* __restrict__ pages, int H, int G, int hd, int rd, int interleaved, int page_size,
                  int heads_per_block) {
    __shared__ float cs[128], sn[128];          // rd / 2 <= 128
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = rd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = (float)pos * inv_freq[i];
        sincosf(angle, &sn[i], &cs[i]);
    }
    __syncthreads();
    const float* src = qkv + (long long)t * ld;
    const int heads = pages ? H + 2 * G : H;
    long long page_base = 0;
    if (pages) {
        const int page = page_table[(long long)seq_ids[t] * pt_stride + pos / page_size];
        page_base = (long long)page * 2 * G * page_size * hd + (long long)(pos % page_size) * hd;
    }
    const int head_begin = blockIdx.y * heads_per_block;
    const int head_end = min(heads, head_begin + heads_per_block);
    // A warp takes whole heads. Rotated heads go pair by pair (each value is read once, both results of a
    // pair are written by the lane that read them); several heads are in flight per lane.
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int rot_end = min(head_end, pages ? H + G : H);          // queries and keys are rotated, values are not
    auto dest = [&](int head, int e) -> long long {
        if (head < H) return ((long long)t * H + head) * hd + e;
        const bool is_v = head >= H + G;
        const int g = is_v ? head - H - G : head - H;
        return page_base + ((long long)(is_v ? G : 0) + g) * page_size * hd + e;
    };
    for (int p = lane; p < half; p += 32) {
        const int a = interleaved ? 2 * p : p, b = interleaved ? 2 * p + 1 : p + half;
        const float c = cs[p], sv = sn[p];
#pragma unroll 4
        for (int head = head_begin + warp; head < rot_end; head += nwarps) {
            const float* hsrc = src + (long long)head * hd;
            const float xa = hsrc[a], xb = hsrc[b];
            // products and sums rounded one by one (no contraction into FMAs): the same bits as the kernel in fours
            const float ra = __fsub_rn(__fmul_rn(xa, c), __fmul_rn(xb, sv)), rb = __fadd_rn(__fmul_rn(xa, sv), __fmul_rn(xb, c));
            if (head < H) {
                q_out[dest(head, a)] = lp_from_float<TQ>(ra);
                q_out[dest(head, b)] = lp_from_float<TQ>(rb);
            } else {
                pages[dest(head, a)] = lp_from_float<TKV>(ra);
                pages[dest(head, b)] = lp_from_float<TKV>(rb);
            }
        }
    }
    // what lies beyond the rotary width passes through
    for (int e = rd + lane; e < hd; e += 32) {
#pragma unroll 4
        for (int head = head_begin + warp; head < rot_end; head += nwarps) {
            const float val = src[(long long)head * hd + e];
            if (head < H) q_out[dest(head, e)] = lp_from_float<TQ>(val);
            else pages[dest(head, e)] = lp_from_float<TKV>(val);
        }
    }
    // values
    const int v_first = max(head_begin, H + G);
    for (int head = v_first + warp; head < head_end; head += nwarps) {
#pragma unroll 4
        for (int e = lane; e < hd; e += 32) pages[dest(head, e)] = lp_from_float<TKV>(src[(long long)head * hd + e]);
    }
}

// The common case in fours: split-half pairs over the whole head (rd == hd, hd a multiple of 8). An item is four
// neighbouring pairs of one head: two float4 loads, one float4 of cosines and of sines, two stores of four values.
template <typename T> __device__ __forceinline__ void store4(T* dst, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* dst, float a, float b, float c, float d) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float a, float b, float c, float d) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
rope_cache_vec_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ inv_freq,
                      const int* __restrict__ positions, const int* __restrict__ seq_ids,
                      const int* __restrict__ page_table, int pt_stride, TQ* __restrict__ q_out,
                      TKV* __restrict__ pages, int H, int G, int hd, int page_size) {
    __shared__ __align__(16) float cs[128], sn[128];
    lp_grid_release();
    lp_grid_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = hd >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
    __syncthreads();
    const float* src = qkv + (long long)t * ld;
    long long page_base = 0;
    if (pages) {
        const int page = page_table[(long long)seq_ids[t] * pt_stride + pos / page_size];
        page_base = (long long)page * 2 * G * page_size * hd + (long long)(pos % page_size) * hd;
    }
    const int qph = half >> 2;                                   // items per rotated head
    const int rot_heads = pages ? H + G : H;
    for (int it = threadIdx.x; it < rot_heads * qph; it += blockDim.x) {
        const int head = it / qph, a = (it - head * qph) * 4;
        const float* hsrc = src + (long long)head * hd;
        const float4 xa = *reinterpret_cast<const float4*>(hsrc + a);
        const float4 xb = *reinterpret_cast<const float4*>(hsrc + a + half);
        const float4 c = *reinterpret_cast<const float4*>(cs + a);
        const float4 sv = *reinterpret_cast<const float4*>(sn + a);
        // products and sums rounded one by one (no contraction into FMAs): the same bits as the kernel above,
        // whichever of the two a step's size selects
#define LP_ROT_A(u) __fsub_rn(__fmul_rn(xa.u, c.u), __fmul_rn(xb.u, sv.u))
#define LP_ROT_B(u) __fadd_rn(__fmul_rn(xa.u, sv.u), __fmul_rn(xb.u, c.u))
        const float ra0 = LP_ROT_A(x), ra1 = LP_ROT_A(y), ra2 = LP_ROT_A(z), ra3 = LP_ROT_A(w);
        const float rb0 = LP_ROT_B(x), rb1 = LP_ROT_B(y), rb2 = LP_ROT_B(z), rb3 = LP_ROT_B(w);
#undef LP_ROT_A
#undef LP_ROT_B
        if (head < H) {
            TQ* dst = q_out + ((long long)t * H + head) * hd + a;
            store4<TQ>(dst, ra0, ra1, ra2, ra3);
            store4<TQ>(dst + half, rb0, rb1, rb2, rb3);
        } else {
            TKV* dst = pages + page_base + (long long)(head - H) * page_size * hd + a;
            store4<TKV>(dst, ra0, ra1, ra2, ra3);
            store4<TKV>(dst + half, rb0, rb1, rb2, rb3);
        }
    }
    if (pages) {                                                 // values: copied as they are
        const int per = hd >> 2;
        for (int it = threadIdx.x; it < G * per; it += blockDim.x) {
            const int g = it / per, e = (it - g * per) * 4;
            const float4 v = *reinterpret_cast<const float4*>(src + (long long)(H + G + g) * hd + e);
            store4<TKV>(pages + page_base + ((long long)G + g) * page_size * hd + e, v.x, v.y, v.z, v.w);
        }
    }
}

extern "C" int lp_rope_cache_write(const float* qkv, int ld, const float* inv_freq, const int* positions,
                                   const int* seq_ids, const int* page_table, int pt_stride, void* q_out,
                                   int q_dtype, void* pages, int kv_dtype, int T, int H, int G, int hd, int rd,
                                   int interleaved, int page_size, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (hd <= 0 || H <= 0 || G < 0) LP_REFUSE("rope_cache_write: heads %d/%d of %d", H, G, hd);
    if (rd < 0 || rd > hd || (rd & 1)) LP_REFUSE("rope_cache_write: rotary width %d of a head of %d", rd, hd);
    if (rd > 256) LP_REFUSE("rope_cache_write: rotary width %d (supported: up to 256)", rd);
    if (rd > 0 && !inv_freq) LP_REFUSE("rope_cache_write: rotation without frequencies");
    const int heads = pages ? H + 2 * G : H;
    if (ld < heads * hd) LP_REFUSE("rope_cache_write: row of %d values for %d heads of %d", ld, heads, hd);
    if (pages && page_size <= 0) LP_REFUSE("rope_cache_write: page size %d", page_size);
    // many tokens, split-half pairs over whole heads of a multiple of 8, everything 16-byte aligned: in fours
    if (T >= 256 && !interleaved && rd == hd && hd % 8 == 0 && ld % 4 == 0 &&
        ((((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)pages) & 15) == 0)) {
#define LP_LAUNCH_ROPE_VEC(TQ, TKV)                                                                         \
    lp_launch(rope_cache_vec_kernel<TQ, TKV>, T, 256, 0, stream, qkv, ld, inv_freq, positions, seq_ids,      \
              page_table, pt_stride, (TQ*)q_out, (TKV*)pages, H, G, hd, page_size)
        if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_ROPE_VEC(float, float);
        else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE_VEC(__nv_bfloat16, __nv_bfloat16);
        else if (q_dtype == LP_F32 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE_VEC(float, __nv_bfloat16);
        else if (q_dtype == LP_BF16 && kv_dtype == LP_F32) LP_LAUNCH_ROPE_VEC(__nv_bfloat16, float);
        else LP_REFUSE("rope_cache_write: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_ROPE_VEC
        return lp_check_launch("rope_cache_write");
    }
    // many tokens: one block per token takes all its heads; few tokens: the heads are shared out
    int heads_per_block = heads;
    if (T < 256) {
        heads_per_block = (512 + hd - 1) / hd;
        if (heads_per_block < 1) heads_per_block = 1;
        if (heads_per_block > heads) heads_per_block = heads;
    }
    const int parts = (heads + heads_per_block - 1) / heads_per_block;
    const int threads = heads_per_block * hd >= 1024 ? 256 : 128;
    dim3 grid(T, parts);
#define LP_LAUNCH_ROPE(TQ, TKV)                                                                          \
    lp_launch(rope_cache_kernel<TQ, TKV>, grid, threads, 0, stream, qkv, ld, inv_freq, positions, seq_ids, \
              page_table, pt_stride, (TQ*)q_out, (TKV*)pages, H, G, hd, rd, interleaved, page_size,       \
              heads_per_block)
    if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_ROPE(float, float);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE(__nv_bfloat16, __nv_bfloat16);
    else if (q_dtype == LP_F32 && kv_dtype == LP_BF16) LP_LAUNCH_ROPE(float, __nv_bfloat16);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_F32) LP_LAUNCH_ROPE(__nv_bfloat16, float);
    else LP_REFUSE("rope_cache_write: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_ROPE
    return lp_check_launch("rope_cache_write");
}

// ---------------------------------------------------------------- layer norm (gain, no bias)
// out[r, i] = (x[row(r), i] - mean) / sqrt(var + eps) * w[i], var = mean of the squared deviations
// from the mean; one block per row, three passes over a row that stays in L1 (sum, squared
// deviations, write), all float32, every sum in a fixed order.
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                 TOut* __restrict__ out, int d, float eps, float* __restrict__ zero, long long zero_count) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int r = blockIdx.x;
    const long long src = rows ? rows[r] : r;
    const float* xr = x + src * d;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) s += xr[i];
    const float mean = lp_block_sum(s, scratch) / (float)d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) {
        const float c = xr[i] - mean;
        ss += c * c;
    }
    const float var = lp_block_sum(ss, scratch) / (float)d;
    const float scale = 1.0f / sqrtf(var + eps);
    TOut* o = out + (long long)r * d;
    for (int i = threadIdx.x; i < d; i += NORM_THREADS) o[i] = lp_from_float<TOut>((xr[i] - mean) * scale * w[i]);
}

// zero (optional): a float32 buffer of zero_count values cleared on the side.
extern "C" int lp_layernorm(const float* x, const int* rows, const float* w, void* out, int out_dtype, int R, int d,
                            float eps, float* zero, long long zero_count, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (d <= 0) LP_REFUSE("layernorm: width %d", d);
    if (out_dtype == LP_F32)
        lp_launch(layernorm_kernel<float>, R, NORM_THREADS, 0, stream, x, rows, w, (float*)out, d, eps, zero, zero_count);
    else if (out_dtype == LP_BF16)
        lp_launch(layernorm_kernel<__nv_bfloat16>, R, NORM_THREADS, 0, stream, x, rows, w, (__nv_bfloat16*)out, d, eps, zero, zero_count);
    else
        LP_REFUSE("layernorm: output dtype code %d", out_dtype);
    return lp_check_launch("layernorm");
}

// ---------------------------------------------------------------- xIELU activation
// act(z) = softplus(p) z^2 + z / 2 for z > 0, (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 otherwise; p and q are
// the two learned numbers `pq` of the layer. z: float32 [T, ldz] (a slice of a wider product), out: [T, F].
__device__ __forceinline__ float lp_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

template <typename TOut>
__global__ void __launch_bounds__(256)
xielu_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ pq, TOut* __restrict__ out, int T, int F,
             float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const float ap = lp_softplus(pq[0]), an = 0.5f + lp_softplus(pq[1]);
    const long long n = (long long)T * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F;
        const int f = (int)(i - t * F);
        const float v = z[t * ldz + f];
        const float a = v > 0.f ? ap * v * v + 0.5f * v : an * (expm1f(v) - v) + 0.5f * v;
        out[i] = lp_from_float<TOut>(a);
    }
}

// The same, four values per thread (rows and row starts of a multiple of four values).
template <typename TOut>
__global__ void __launch_bounds__(256)
xielu_vec4_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ pq, TOut* __restrict__ out, int T, int F,
                  float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const float ap = lp_softplus(pq[0]), an = 0.5f + lp_softplus(pq[1]);
    const int quads = F >> 2;
    const long long n = (long long)T * quads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / quads;
        const int f = (int)(i - t * quads) * 4;
        const float4 v = *reinterpret_cast<const float4*>(z + t * ldz + f);
        float a[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) a[k] = a[k] > 0.f ? ap * a[k] * a[k] + 0.5f * a[k] : an * (expm1f(a[k]) - a[k]) + 0.5f * a[k];
        TOut* o = out + t * F + f;
        if (sizeof(TOut) == 2) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(a[0], a[1]), hi = __floats2bfloat162_rn(a[2], a[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(o) = packed;
        } else {
            *reinterpret_cast<float4*>(o) = make_float4(a[0], a[1], a[2], a[3]);
        }
    }
}

// zero (optional): a float32 buffer of zero_count values cleared on the side, for the product after the activation when
// it sums partial results into its output.
extern "C" int lp_xielu(const float* z, int ldz, const float* pq, void* out, int out_dtype, int T, int F, float* zero,
                        long long zero_count, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return 0;
    if (ldz < F) LP_REFUSE("xielu: rows of %d values for %d features", ldz, F);
    if (F % 4 == 0 && ldz % 4 == 0 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0) {
        const long long n4 = (long long)T * (F / 4);
        long long blocks4 = (n4 + 255) / 256;
        if (blocks4 > 148 * 16) blocks4 = 148 * 16;
        if (out_dtype == LP_F32) lp_launch(xielu_vec4_kernel<float>, (unsigned)blocks4, 256, 0, stream, z, ldz, pq, (float*)out, T, F, zero, zero_count);
        else if (out_dtype == LP_BF16)
            lp_launch(xielu_vec4_kernel<__nv_bfloat16>, (unsigned)blocks4, 256, 0, stream, z, ldz, pq, (__nv_bfloat16*)out, T, F, zero, zero_count);
        else LP_REFUSE("xielu: output dtype code %d", out_dtype);
        return lp_check_launch("xielu");
    }
    const long long n = (long long)T * F;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == LP_F32) lp_launch(xielu_kernel<float>, (unsigned)blocks, 256, 0, stream, z, ldz, pq, (float*)out, T, F, zero, zero_count);
    else if (out_dtype == LP_BF16)
        lp_launch(xielu_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, z, ldz, pq, (__nv_bfloat16*)out, T, F, zero, zero_count);
    else LP_REFUSE("xielu: output dtype code %d", out_dtype);
    return lp_check_launch("xielu");
}

// ---------------------------------------------------------------- gated residual sum and weighted sum over depth
// y[t, i] = x[t, i] + a[t, i] * sigmoid(ga[t, i] + ba[i]) + b[t, i] * sigmoid(gb[t, i] + bb[i])
// (a gate pointer that is null leaves its branch ungated, a branch pointer that is null leaves it out), all float32.
// With `streams` [count, T, d]: y is kept as stream `count - 1`, and x <- sum_j mix[j] * streams[j] over
// j = 0 .. count - 1 in increasing j; without, x <- y. `keep_input`: the incoming x is stream `count - 2` and is
// stored there first (the first layer of a model, whose input is the embedding's output).
__global__ void __launch_bounds__(256)
gated_sum_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ ga, int ldga,
                 const float* __restrict__ ba, const float* __restrict__ b, const float* __restrict__ gb, int ldgb,
                 const float* __restrict__ bb, float* __restrict__ streams, const float* __restrict__ mix, int count,
                 int keep_input, int T, int d) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / d;
        const int c = (int)(i - t * d);
        float y = x[i];
        if (streams && keep_input) streams[(long long)(count - 2) * n + i] = y;
        if (a) {
            float v = a[i];
            if (ga) v *= 1.0f / (1.0f + expf(-(ga[t * ldga + c] + (ba ? ba[c] : 0.f))));
            y += v;
        }
        if (b) {
            float v = b[i];
            if (gb) v *= 1.0f / (1.0f + expf(-(gb[t * ldgb + c] + (bb ? bb[c] : 0.f))));
            y += v;
        }
        if (streams) {
            streams[(long long)(count - 1) * n + i] = y;
            float s = 0.f;
            for (int j = 0; j + 1 < count; ++j) s = fmaf(mix[j], streams[(long long)j * n + i], s);
            y = fmaf(mix[count - 1], y, s);
        }
        x[i] = y;
    }
}

extern "C" int lp_gated_sum(float* x, const float* a, const float* ga, int ldga, const float* ba, const float* b,
                            const float* gb, int ldgb, const float* bb, float* streams, const float* mix, int count,
                            int keep_input, int T, int d, cudaStream_t stream) {
    if (T <= 0 || d <= 0) return 0;
    if (streams && (count < 1 || !mix)) LP_REFUSE("gated_sum: %d streams without weights", count);
    if (streams && keep_input && count < 2) LP_REFUSE("gated_sum: no place for the input among %d streams", count);
    const long long n = (long long)T * d;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    lp_launch(gated_sum_kernel, (unsigned)blocks, 256, 0, stream, x, a, ga, ldga, ba, b, gb, ldgb, bb, streams, mix, count, keep_input, T, d);
    return lp_check_launch("gated_sum");
}

// ---------------------------------------------------------------- rotation angles of a step's tokens
// out[t][i] = (cos, sin) of float(positions[t]) * inv_freq[i]: the same float32 product and the same sincosf as
// the rotation kernels above, formed once per step for a product whose epilogue rotates (gemm_tcgen05.cu).
__global__ void __launch_bounds__(128)
rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq, float2* __restrict__ out,
                   int T, int half) {
    lp_grid_release();
    lp_grid_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T * half) return;
    const int t = (int)(i / half), p = (int)(i - (long long)t * half);
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[p], &sn, &cs);
    out[i] = make_float2(cs, sn);
}

extern "C" int lp_rope_angles(const int* positions, const float* inv_freq, float* out, int T, int half,
                              cudaStream_t stream) {
    if (T <= 0 || half <= 0) return 0;
    const long long n = (long long)T * half;
    lp_launch(rope_angles_kernel, (unsigned)((n + 127) / 128), 128, 0, stream, positions, inv_freq, (float2*)out, T, half);
    return lp_check_launch("rope_angles");
}

// ---------------------------------------------------------------- advancing a decoding batch on the device
// After a decode step whose sampler left one token per sequence: that token becomes the next
// step's input, and every sequence moves on by one position. Lets decode steps follow one
// another without the host (the reference keeps position and length on the device for the
// same reason: java21 inference/CudaForwardPass.java:138-141).
__global__ void advance_kernel(int* __restrict__ tokens, int* __restrict__ positions, int* __restrict__ kv_len,
                               const int* __restrict__ sampled, int B) {
    lp_grid_release();
    lp_grid_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < B) {
        tokens[i] = sampled[i];
        positions[i] += 1;
        kv_len[i] += 1;
    }
}

extern "C" int lp_advance(int* tokens, int* positions, int* kv_len, const int* sampled, int B, cudaStream_t stream) {
    if (B <= 0) return 0;
    lp_launch(advance_kernel, (B + 127) / 128, 128, 0, stream, tokens, positions, kv_len, sampled, B);
    return lp_check_launch("advance");
}

// ---------------------------------------------------------------- queries, keys and values of a general attention layer
// One block per token of the fused projection output
//   qkv[t] = [ H query heads x dk | G key heads x dk | G value heads x dv ]   (float32),
// for layers whose heads need more than a rotation: an additive bias per feature (`bias`, optional), the rotation of
// the first `rd` features of every query and key head (pairs (2i, 2i+1) or (i, i + rd/2); angle = float(position) *
// inv_freq[pair]; the pair (u, v) becomes (u cos - v sin, v cos + u sin)), and then (`unit`) the division of every
// query and key head by its root mean square over dk, with `unit_eps` inside the root. Keys and values may differ in
// size: queries, keys and values are stored with `hdp` features per head (hdp >= dk, dv), the rest zero, so that the
// attention kernels see one head size; queries go to q_out[t, h, :hdp], keys and values to the page of the token's
// sequence that holds its position, pages[page][0|1][g][position % page_size][:hdp]. A warp per head; all float32.
// `qgain` / `kgain` (optional, [dk], shared by the heads): BEFORE the rotation every query / key head is RMS-normed
// over dk with that gain and `gain_eps` inside the root. G = 0 with `pages` null: a layer that has queries only.
constexpr int PREP_MAX = 256;
template <typename TQ, typename TKV>
__global__ void __launch_bounds__(256)
qkv_prepare_kernel(const float* __restrict__ qkv, int ld, const float* __restrict__ bias, const float* __restrict__ inv_freq,
                   const int* __restrict__ positions, const int* __restrict__ seq_ids, const int* __restrict__ page_table,
                   int pt_stride, TQ* __restrict__ q_out, TKV* __restrict__ pages, int H, int G, int dk, int dv, int hdp,
                   int rd, int interleaved, int unit, float unit_eps, int page_size, float* __restrict__ zero,
                   long long zero_count, const float* __restrict__ qgain, const float* __restrict__ kgain, float gain_eps) {
    __shared__ float cs[PREP_MAX];
    __shared__ float buf[8][PREP_MAX];
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int pos = positions[t];
    const int half = rd >> 1;
    for (int i = tid; i < half; i += blockDim.x) {
        float s, c;
        sincosf((float)pos * inv_freq[i], &s, &c);
        cs[2 * i] = c;
        cs[2 * i + 1] = s;
    }
    __syncthreads();
    const float* row = qkv + (long long)t * ld;
    const long long page = G > 0 ? page_table[(long long)seq_ids[t] * pt_stride + pos / page_size] : 0;
    const int r = pos % page_size;
    for (int item = warp; item < H + 2 * G; item += 8) {
        if (item < H + G) {
            const int src = item * dk;               // query heads, then key heads, lie one after another
            const float* gain = item < H ? qgain : kgain;
            float pre = 1.0f;
            if (gain) {
                float s0 = 0.f;
                for (int e = lane; e < dk; e += 32) {
                    const float val = row[src + e] + (bias ? bias[src + e] : 0.f);
                    s0 += val * val;
                }
                pre = 1.0f / sqrtf(lp_warp_sum(s0) / (float)dk + gain_eps);
            }
            float ss = 0.f;
            for (int e = lane; e < dk; e += 32) {
                float val = row[src + e] + (bias ? bias[src + e] : 0.f);
                if (gain) val = val * pre * gain[e];
                if (e < rd) {
                    int pair, partner;
                    bool first;
                    if (interleaved) { pair = e >> 1; first = !(e & 1); partner = e ^ 1; }
                    else { first = e < half; pair = first ? e : e - half; partner = first ? e + half : e - half; }
                    float other = row[src + partner] + (bias ? bias[src + partner] : 0.f);
                    if (gain) other = other * pre * gain[partner];
                    const float c = cs[2 * pair], s = cs[2 * pair + 1];
                    val = first ? val * c - other * s : val * c + other * s;
                }
                buf[warp][e] = val;
                ss += val * val;
            }
            ss = lp_warp_sum(ss);
            const float factor = unit ? 1.0f / sqrtf(ss / (float)dk + unit_eps) : 1.0f;
            __syncwarp();
            if (item < H) {
                TQ* dst = q_out + ((long long)t * H + item) * hdp;
                for (int e = lane; e < hdp; e += 32) dst[e] = lp_from_float<TQ>(e < dk ? buf[warp][e] * factor : 0.f);
            } else {
                TKV* dst = pages + (((page * 2 + 0) * G + (item - H)) * page_size + r) * hdp;
                for (int e = lane; e < hdp; e += 32) dst[e] = lp_from_float<TKV>(e < dk ? buf[warp][e] * factor : 0.f);
            }
            __syncwarp();
        } else {
            const int g = item - H - G;
            const int src = (H + G) * dk + g * dv;
            TKV* dst = pages + (((page * 2 + 1) * G + g) * page_size + r) * hdp;
            for (int e = lane; e < hdp; e += 32)
                dst[e] = lp_from_float<TKV>(e < dv ? row[src + e] + (bias ? bias[src + e] : 0.f) : 0.f);
        }
    }
}

extern "C" int lp_qkv_prepare(const float* qkv, int ld, const float* bias, const float* inv_freq, const int* positions,
                              const int* seq_ids, const int* page_table, int pt_stride, void* q_out, int q_dtype,
                              void* pages, int kv_dtype, int T, int H, int G, int dk, int dv, int hdp, int rd,
                              int interleaved, int unit, float unit_eps, int page_size, float* zero, long long zero_count,
                              const float* qgain, const float* kgain, float gain_eps, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G < 0 || dk <= 0 || dv <= 0) LP_REFUSE("qkv_prepare: %d / %d heads of %d and %d", H, G, dk, dv);
    if (hdp < dk || hdp < dv || dk > PREP_MAX) LP_REFUSE("qkv_prepare: heads of %d and %d stored in %d (at most %d)", dk, dv, hdp, PREP_MAX);
    if (rd < 0 || rd > dk || (rd & 1)) LP_REFUSE("qkv_prepare: rotary width %d for heads of %d", rd, dk);
    if (rd > 0 && !inv_freq) LP_REFUSE("qkv_prepare: a rotation without frequencies");
    if (ld < (H + G) * dk + G * dv) LP_REFUSE("qkv_prepare: rows of %d values for %d", ld, (H + G) * dk + G * dv);
    if (G > 0 && (page_size <= 0 || !pages)) LP_REFUSE("qkv_prepare: needs the pages of the cache");
    if (G == 0) page_size = 1;
#define LP_LAUNCH_PREP(TQ, TKV)                                                                                       \
    lp_launch(qkv_prepare_kernel<TQ, TKV>, T, 256, 0, stream, qkv, ld, bias, inv_freq, positions, seq_ids, page_table, \
              pt_stride, (TQ*)q_out, (TKV*)pages, H, G, dk, dv, hdp, rd, interleaved, unit, unit_eps, page_size, zero,  \
              zero_count, qgain, kgain, gain_eps)
    if (q_dtype == LP_F32 && kv_dtype == LP_F32) LP_LAUNCH_PREP(float, float);
    else if (q_dtype == LP_BF16 && kv_dtype == LP_BF16) LP_LAUNCH_PREP(__nv_bfloat16, __nv_bfloat16);
    else LP_REFUSE("qkv_prepare: dtype codes q=%d kv=%d", q_dtype, kv_dtype);
#undef LP_LAUNCH_PREP
    return lp_check_launch("qkv_prepare");
}

// ---------------------------------------------------------------- norm of a sublayer's result, residual sum, next norm
// x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w   (the norm that follows a sublayer, then the residual sum), and, when
// `w2` is given, out2[t] = x[t] / sqrt(mean(x[t]^2) + eps2) * w2 (the norm in front of the next sublayer) in the same
// pass. One block per row; float32; sums in a fixed order. Optional: `ybias` [d] is added to y first (the additive
// vector of the sublayer's last map); `scale` [d] multiplies the normed result once more (a layer scale); `out2` without
// `w2` receives the new x as it is (for a next sublayer that reads the stream itself, in its own number format).
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
post_norm_add_kernel(const float* __restrict__ y, const float* __restrict__ w, float eps, float* __restrict__ x,
                     const float* __restrict__ w2, float eps2, TOut* __restrict__ out2, int d, float* __restrict__ zero,
                     long long zero_count, const float* __restrict__ ybias, const float* __restrict__ scale) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long row = blockIdx.x;
    const float* yr = y + row * d;
    float* xr = x + row * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = yr[i] + (ybias ? ybias[i] : 0.f);
        ss += v * v;
    }
    ss = lp_block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)d + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float add = (yr[i] + (ybias ? ybias[i] : 0.f)) * f * w[i];
        if (scale) add *= scale[i];
        const float v = xr[i] + add;
        xr[i] = v;
        ss2 += v * v;
        if (!w2 && out2) out2[row * d + i] = lp_from_float<TOut>(v);
    }
    if (!w2) return;
    ss2 = lp_block_sum(ss2, scratch);
    const float f2 = 1.0f / sqrtf(ss2 / (float)d + eps2);
    TOut* o = out2 + row * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = lp_from_float<TOut>(xr[i] * f2 * w2[i]);
}

// The same for rows of a multiple of four values: four values per load and store.
template <typename TOut>
__global__ void __launch_bounds__(NORM_THREADS)
post_norm_add_vec4_kernel(const float* __restrict__ y, const float* __restrict__ w, float eps, float* __restrict__ x,
                          const float* __restrict__ w2, float eps2, TOut* __restrict__ out2, int d, float* __restrict__ zero,
                          long long zero_count, const float* __restrict__ ybias, const float* __restrict__ scale) {
    __shared__ float scratch[32];
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long row = blockIdx.x;
    const float4* yr = reinterpret_cast<const float4*>(y + row * d);
    float4* xr = reinterpret_cast<float4*>(x + row * d);
    const float4* wr = reinterpret_cast<const float4*>(w);
    const float4* br = reinterpret_cast<const float4*>(ybias);
    const float4* sr = reinterpret_cast<const float4*>(scale);
    const int quads = d >> 2;
    float ss = 0.f;
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        float4 v = yr[i];
        if (br) { const float4 b = br[i]; v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    ss = lp_block_sum(ss, scratch);
    const float f = 1.0f / sqrtf(ss / (float)d + eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        float4 v = yr[i];
        const float4 g = wr[i];
        if (br) { const float4 b = br[i]; v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w; }
        float4 a = make_float4(v.x * f * g.x, v.y * f * g.y, v.z * f * g.z, v.w * f * g.w);
        if (sr) { const float4 c = sr[i]; a.x *= c.x; a.y *= c.y; a.z *= c.z; a.w *= c.w; }
        float4 r = xr[i];
        r.x += a.x; r.y += a.y; r.z += a.z; r.w += a.w;
        xr[i] = r;
        ss2 += r.x * r.x + r.y * r.y + r.z * r.z + r.w * r.w;
        if (!w2 && out2) store4<TOut>(out2 + row * d + 4 * i, r.x, r.y, r.z, r.w);
    }
    if (!w2) return;
    ss2 = lp_block_sum(ss2, scratch);
    const float f2 = 1.0f / sqrtf(ss2 / (float)d + eps2);
    const float4* w2r = reinterpret_cast<const float4*>(w2);
    TOut* o = out2 + row * d;
    for (int i = threadIdx.x; i < quads; i += blockDim.x) {
        const float4 r = xr[i], g = w2r[i];
        store4<TOut>(o + 4 * i, r.x * f2 * g.x, r.y * f2 * g.y, r.z * f2 * g.z, r.w * f2 * g.w);
    }
}

extern "C" int lp_post_norm_add(const float* y, const float* w, float eps, float* x, const float* w2, float eps2,
                                void* out2, int out2_dtype, int T, int d, float* zero, long long zero_count,
                                const float* ybias, const float* scale, cudaStream_t stream) {
    if (T <= 0 || d <= 0) return 0;
    if (w2 && !out2) LP_REFUSE("post_norm_add: a second norm without its output");
    if (d % 4 == 0 && (((uintptr_t)y | (uintptr_t)x | (uintptr_t)w | (uintptr_t)w2 | (uintptr_t)out2 | (uintptr_t)ybias | (uintptr_t)scale) & 15) == 0) {
        if (!out2 || out2_dtype == LP_F32)
            lp_launch(post_norm_add_vec4_kernel<float>, T, NORM_THREADS, 0, stream, y, w, eps, x, w2, eps2, (float*)out2, d, zero, zero_count, ybias, scale);
        else if (out2_dtype == LP_BF16)
            lp_launch(post_norm_add_vec4_kernel<__nv_bfloat16>, T, NORM_THREADS, 0, stream, y, w, eps, x, w2, eps2, (__nv_bfloat16*)out2, d, zero, zero_count, ybias, scale);
        else LP_REFUSE("post_norm_add: output dtype code %d", out2_dtype);
        return lp_check_launch("post_norm_add");
    }
    if (!out2 || out2_dtype == LP_F32)
        lp_launch(post_norm_add_kernel<float>, T, NORM_THREADS, 0, stream, y, w, eps, x, w2, eps2, (float*)out2, d, zero, zero_count, ybias, scale);
    else if (out2_dtype == LP_BF16)
        lp_launch(post_norm_add_kernel<__nv_bfloat16>, T, NORM_THREADS, 0, stream, y, w, eps, x, w2, eps2, (__nv_bfloat16*)out2, d, zero, zero_count, ybias, scale);
    else LP_REFUSE("post_norm_add: output dtype code %d", out2_dtype);
    return lp_check_launch("post_norm_add");
}

// ---------------------------------------------------------------- additions to the stream between runs of layers
// x[t, i] += other[t, i] + vec[i]; either may be absent. float32.
__global__ void __launch_bounds__(256)
stream_add_kernel(float* __restrict__ x, const float* __restrict__ other, const float* __restrict__ vec, int T, int d) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i];
        if (other) v += other[i];
        if (vec) v += vec[i % d];
        x[i] = v;
    }
}

extern "C" int lp_stream_add(float* x, const float* other, const float* vec, int T, int d, cudaStream_t stream) {
    if (T <= 0 || d <= 0 || (!other && !vec)) return 0;
    const long long n = (long long)T * d;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    lp_launch(stream_add_kernel, (unsigned)blocks, 256, 0, stream, x, other, vec, T, d);
    return lp_check_launch("stream_add");
}

// ---------------------------------------------------------------- squared ReLU
// out[t, f] = max(z[t, f], 0)^2 on the float32 sums of an up projection (z: [T, ldz], may be a slice).
template <typename TOut>
__global__ void __launch_bounds__(256)
relu2_kernel(const float* __restrict__ z, int ldz, TOut* __restrict__ out, int T, int F, float* __restrict__ zero,
             long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long n = (long long)T * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F;
        const float v = fmaxf(z[t * ldz + (i - t * F)], 0.f);
        out[i] = lp_from_float<TOut>(v * v);
    }
}

// The same, four values per thread (rows and row starts of a multiple of four values).
template <typename TOut>
__global__ void __launch_bounds__(256)
relu2_vec4_kernel(const float* __restrict__ z, int ldz, TOut* __restrict__ out, int T, int F, float* __restrict__ zero,
                  long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int quads = F >> 2;
    const long long n = (long long)T * quads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / quads;
        const int f = (int)(i - t * quads) * 4;
        const float4 v = *reinterpret_cast<const float4*>(z + t * ldz + f);
        const float a = fmaxf(v.x, 0.f), b = fmaxf(v.y, 0.f), c = fmaxf(v.z, 0.f), d = fmaxf(v.w, 0.f);
        store4<TOut>(out + t * F + f, a * a, b * b, c * c, d * d);
    }
}

extern "C" int lp_relu2(const float* z, int ldz, void* out, int out_dtype, int T, int F, float* zero, long long zero_count,
                        cudaStream_t stream) {
    if (T <= 0 || F <= 0) return 0;
    if (ldz < F) LP_REFUSE("relu2: rows of %d values for %d features", ldz, F);
    if (F % 4 == 0 && ldz % 4 == 0 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0) {
        const long long n4 = (long long)T * (F / 4);
        long long blocks4 = (n4 + 255) / 256;
        if (blocks4 > 148 * 16) blocks4 = 148 * 16;
        if (out_dtype == LP_F32) lp_launch(relu2_vec4_kernel<float>, (unsigned)blocks4, 256, 0, stream, z, ldz, (float*)out, T, F, zero, zero_count);
        else if (out_dtype == LP_BF16) lp_launch(relu2_vec4_kernel<__nv_bfloat16>, (unsigned)blocks4, 256, 0, stream, z, ldz, (__nv_bfloat16*)out, T, F, zero, zero_count);
        else LP_REFUSE("relu2: output dtype code %d", out_dtype);
        return lp_check_launch("relu2");
    }
    const long long n = (long long)T * F;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == LP_F32) lp_launch(relu2_kernel<float>, (unsigned)blocks, 256, 0, stream, z, ldz, (float*)out, T, F, zero, zero_count);
    else if (out_dtype == LP_BF16) lp_launch(relu2_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, z, ldz, (__nv_bfloat16*)out, T, F, zero, zero_count);
    else LP_REFUSE("relu2: output dtype code %d", out_dtype);
    return lp_check_launch("relu2");
}

// ---------------------------------------------------------------- gated activation of a dense feed-forward
// out[t, f] = act(z[t, f] + b[f]) * (z[t, F + f] + b[F + f]) from the float32 sums of a stacked gate | up product
// (z: rows of ldz values, the F gate sums first, then the F up sums; b: [2 F] or null). act: the tanh form of GELU,
//     0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))),
// evaluated in float32 (form 0), or the logistic form g / (1 + exp(-g)) (form 1).
__device__ __forceinline__ float lp_gated_value(float g, float u, int form) {
    if (form == 0) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    return g / (1.0f + expf(-g)) * u;
}

template <typename TOut>
__global__ void __launch_bounds__(256)
gated_act_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, TOut* __restrict__ out, int T, int F,
                 int form, float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long n = (long long)T * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / F;
        const int f = (int)(i - t * F);
        const float g = z[t * ldz + f] + (bias ? bias[f] : 0.f);
        const float u = z[t * ldz + F + f] + (bias ? bias[F + f] : 0.f);
        out[i] = lp_from_float<TOut>(lp_gated_value(g, u, form));
    }
}

// The same, four values per thread (F and ldz multiples of four, 16-byte aligned pointers).
template <typename TOut>
__global__ void __launch_bounds__(256)
gated_act_vec4_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, TOut* __restrict__ out, int T,
                      int F, int form, float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const int quads = F >> 2;
    const long long n = (long long)T * quads;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / quads;
        const int f = (int)(i - t * quads) * 4;
        float4 g = *reinterpret_cast<const float4*>(z + t * ldz + f);
        float4 u = *reinterpret_cast<const float4*>(z + t * ldz + F + f);
        if (bias) {
            const float4 bg = *reinterpret_cast<const float4*>(bias + f), bu = *reinterpret_cast<const float4*>(bias + F + f);
            g.x += bg.x; g.y += bg.y; g.z += bg.z; g.w += bg.w;
            u.x += bu.x; u.y += bu.y; u.z += bu.z; u.w += bu.w;
        }
        store4<TOut>(out + t * F + f, lp_gated_value(g.x, u.x, form), lp_gated_value(g.y, u.y, form),
                     lp_gated_value(g.z, u.z, form), lp_gated_value(g.w, u.w, form));
    }
}

extern "C" int lp_gated_act(const float* z, int ldz, const float* bias, void* out, int out_dtype, int T, int F, int form,
                            float* zero, long long zero_count, cudaStream_t stream) {
    if (T <= 0 || F <= 0) return 0;
    if (ldz < 2 * F) LP_REFUSE("gated_act: rows of %d values for %d gate and %d up sums", ldz, F, F);
    if (form < 0 || form > 1) LP_REFUSE("gated_act: form %d", form);
    if (out_dtype != LP_F32 && out_dtype != LP_BF16) LP_REFUSE("gated_act: output dtype code %d", out_dtype);
    const bool vec = F % 4 == 0 && ldz % 4 == 0 && (((uintptr_t)z | (uintptr_t)out | (uintptr_t)bias) & 15) == 0;
    const long long n = vec ? (long long)T * (F / 4) : (long long)T * F;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (vec) {
        if (out_dtype == LP_F32) lp_launch(gated_act_vec4_kernel<float>, (unsigned)blocks, 256, 0, stream, z, ldz, bias, (float*)out, T, F, form, zero, zero_count);
        else lp_launch(gated_act_vec4_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, z, ldz, bias, (__nv_bfloat16*)out, T, F, form, zero, zero_count);
    } else {
        if (out_dtype == LP_F32) lp_launch(gated_act_kernel<float>, (unsigned)blocks, 256, 0, stream, z, ldz, bias, (float*)out, T, F, form, zero, zero_count);
        else lp_launch(gated_act_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, z, ldz, bias, (__nv_bfloat16*)out, T, F, form, zero, zero_count);
    }
    return lp_check_launch("gated_act");
}

// ---------------------------------------------------------------- the stream in another number format
// out[i] = x[i] for n float32 values (a sublayer that reads the stream itself takes it in its own format).
template <typename TOut>
__global__ void __launch_bounds__(256)
stream_cast_kernel(const float* __restrict__ x, TOut* __restrict__ out, long long n, float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = lp_from_float<TOut>(x[i]);
}

extern "C" int lp_stream_cast(const float* x, void* out, int out_dtype, long long n, float* zero, long long zero_count,
                              cudaStream_t stream) {
    if (n <= 0) return 0;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (out_dtype == LP_F32) lp_launch(stream_cast_kernel<float>, (unsigned)blocks, 256, 0, stream, x, (float*)out, n, zero, zero_count);
    else if (out_dtype == LP_BF16) lp_launch(stream_cast_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, x, (__nv_bfloat16*)out, n, zero, zero_count);
    else LP_REFUSE("stream_cast: output dtype code %d", out_dtype);
    return lp_check_launch("stream_cast");
}

// ---------------------------------------------------------------- two sublayers' results summed with constants
// x[t, i] += sa * (a[t, i] + va[i]) + sb * (b[t, i] + vb[i]); b, va and vb may be absent. float32.
__global__ void __launch_bounds__(256)
scaled_sum_kernel(float* __restrict__ x, const float* __restrict__ a, const float* __restrict__ va, float sa,
                  const float* __restrict__ b, const float* __restrict__ vb, float sb, int T, int d) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % d);
        float v = x[i];
        v = fmaf(sa, a[i] + (va ? va[c] : 0.f), v);
        if (b) v = fmaf(sb, b[i] + (vb ? vb[c] : 0.f), v);
        x[i] = v;
    }
}

extern "C" int lp_scaled_sum(float* x, const float* a, const float* va, float sa, const float* b, const float* vb, float sb,
                             int T, int d, cudaStream_t stream) {
    if (T <= 0 || d <= 0) return 0;
    const long long n = (long long)T * d;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    lp_launch(scaled_sum_kernel, (unsigned)blocks, 256, 0, stream, x, a, va, sa, b, vb, sb, T, d);
    return lp_check_launch("scaled_sum");
}
