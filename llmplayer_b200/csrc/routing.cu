// Routing of a mixture of experts: from the router's logits of every token to a weight per expert, and the scaling of
// the experts' hidden activations by those weights.
//
//   score s[e] = sigmoid(z[e])
//   the experts form `groups` equal groups of neighbours; a group's score is the sum of its two largest scores
//   (of its only score, in groups of one); only experts of the `keep` best groups may be chosen
//   the `top` experts with the largest scores among those are chosen; weight = s[e] / (sum of the chosen s + 1e-20)
//
// The experts themselves are run as one stacked gated product over all experts (every token through every expert)
// whose hidden activations are multiplied by the token's weight for that expert (zero for experts it did not choose)
// before one stacked down product sums them; `lp_expert_scale` is that multiplication.
// Among equal scores the expert (group) with the lower index wins. Everything is float32.
#include "common.cuh"

namespace {

// A warp per token. Shared memory per warp: s[E], allowed/chosen flags[E] (as float), group scores[groups].
__global__ void __launch_bounds__(128)
route_kernel(const float* __restrict__ z, int ldz, float* __restrict__ weights, int ldw, int T, int E, int groups,
             int keep, int top) {
    extern __shared__ float sm[];
    lp_grid_release();
    lp_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * (2 * E + groups);
    float* flag = s + E;
    float* gs = flag + E;
    const int per = E / groups;
    for (int e = lane; e < E; e += 32) {
        s[e] = 1.0f / (1.0f + expf(-z[t * ldz + e]));
        flag[e] = 0.f;
    }
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
        float a = -1.f, b = -1.f;                       // the two largest scores of the group (scores are >= 0)
        for (int j = 0; j < per; ++j) {
            const float v = s[g * per + j];
            if (v > a) { b = a; a = v; }
            else if (v > b) b = v;
        }
        gs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    if (lane == 0) {
        for (int n = 0; n < keep; ++n) {                // the best groups, one after another
            int best = -1;
            float bv = -INFINITY;
            for (int g = 0; g < groups; ++g)
                if (gs[g] > bv) { bv = gs[g]; best = g; }
            if (best < 0) break;
            gs[best] = -INFINITY;
            for (int j = 0; j < per; ++j) flag[best * per + j] = 1.f;     // 1: may be chosen
        }
        float sum = 0.f;
        for (int n = 0; n < top; ++n) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (flag[e] == 1.f && s[e] > bv) { bv = s[e]; best = e; }
            if (best < 0) break;
            flag[best] = 2.f;                            // 2: chosen
            sum += bv;
        }
        gs[0] = 1.0f / (sum + 1e-20f);
    }
    __syncwarp();
    const float inv = gs[0];
    for (int e = lane; e < E; e += 32) weights[t * ldw + e] = flag[e] == 2.f ? s[e] * inv : 0.f;
}

// hidden[t, c] *= weights[t, c / ff] for c < E * ff (in place; the columns beyond belong to experts every token uses)
// Experts that are the identity ride along in the same launch: x[t, :] += h[t, :] * sum of the token's weights for them
// (columns first .. first + count - 1 of the weights). x: float32 [T, d], the stream the experts' outputs are added to
// by the product that follows; h: the feed-forward's input [T, d].
struct IdentityShare {
    float* x;
    const void* h;
    int h_bf16, first, count, d;
};
__device__ __forceinline__ void add_identity_share(const IdentityShare& id, const float* __restrict__ weights, int ldw, long long t,
                                                   int begin, int stride) {
    float w = 0.f;
    for (int e = 0; e < id.count; ++e) w += weights[t * ldw + id.first + e];
    if (w == 0.f) return;
    for (int i = begin; i < id.d; i += stride) {
        const float hv = id.h_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(id.h)[t * id.d + i])
                                   : reinterpret_cast<const float*>(id.h)[t * id.d + i];
        id.x[t * id.d + i] = fmaf(hv, w, id.x[t * id.d + i]);
    }
}

template <typename TH>
__global__ void __launch_bounds__(256)
expert_scale_kernel(TH* __restrict__ hidden, int ldh, const float* __restrict__ weights, int ldw, int T, int E, int ff,
                    float* __restrict__ zero, long long zero_count, IdentityShare id) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    if (id.x)                                    // a block per token at a time
        for (long long t = blockIdx.x; t < T; t += gridDim.x) add_identity_share(id, weights, ldw, t, threadIdx.x, blockDim.x);
    const long long cols = (long long)E * ff;
    const long long n = (long long)T * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / cols;
        const int c = (int)(i - t * cols);
        TH* at = hidden + t * ldh + c;
        *at = lp_from_float<TH>(lp_to_float(*at) * weights[t * ldw + c / ff]);
    }
}

// The same, eight bfloat16 columns of one expert per thread (expert sizes and rows of a multiple of eight values).
__global__ void __launch_bounds__(256)
expert_scale_vec8_kernel(__nv_bfloat16* __restrict__ hidden, int ldh, const float* __restrict__ weights, int ldw, int E, int ff,
                         float* __restrict__ zero, long long zero_count, IdentityShare id) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long t = blockIdx.y;
    if (id.x) add_identity_share(id, weights, ldw, t, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
    const int octets = E * ff / 8;
    for (int o = blockIdx.x * blockDim.x + threadIdx.x; o < octets; o += gridDim.x * blockDim.x) {
        const int c = o * 8;
        const float w = weights[t * ldw + c / ff];
        uint4* at = reinterpret_cast<uint4*>(hidden + t * ldh + c);
        uint4 v = *at;
        __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(pairs[k]);
            pairs[k] = __floats2bfloat162_rn(f.x * w, f.y * w);
        }
        *at = v;
    }
}


// Another rule: the `top` experts with the largest logits z[e] + bias[e] are chosen, and their weights are the softmax
// over the chosen logits alone. A warp per token; among equal logits the expert with the lower index wins. `extra`
// further columns of z (beyond the E logits) are gates of experts that every token uses: weights[t, E + i] =
// sigmoid(z[t, E + i]).
__global__ void __launch_bounds__(128)
route_top_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ bias, float* __restrict__ weights, int ldw,
                 int T, int E, int top, int extra) {
    extern __shared__ float sm[];
    lp_grid_release();
    lp_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * 2 * E;
    float* w = s + E;
    for (int e = lane; e < E; e += 32) {
        s[e] = z[t * ldz + e] + (bias ? bias[e] : 0.f);
        w[e] = 0.f;
    }
    __syncwarp();
    float big = 0.f, sum = 0.f;
    for (int n = 0; n < top; ++n) {
        // the largest logit not yet chosen: each lane over its experts, then over the lanes (lower index wins a tie)
        float bv = -INFINITY;
        int best = E;
        for (int e = lane; e < E; e += 32)
            if (w[e] == 0.f && s[e] > bv) { bv = s[e]; best = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best, o);
            if (ov > bv || (ov == bv && oe < best)) { bv = ov; best = oe; }
        }
        if (best >= E) break;
        if (n == 0) big = bv;
        const float p = expf(bv - big);
        sum += p;
        if (lane == 0) w[best] = p;
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) weights[t * ldw + e] = w[e] * inv;
    for (int i = lane; i < extra; i += 32) weights[t * ldw + E + i] = 1.0f / (1.0f + expf(-z[t * ldz + E + i]));
}

// Hidden activations of clamped gated experts from the float32 sums of ONE stacked product over all experts:
// z[t] = [ gate sums of all experts (total) | up sums of all experts (total) ]. With g = min(gate, limit) and
// u = clamp(up, -limit, limit):  hidden[t, c] = g * sigmoid(1.702 g) * (u + 1) * weights[t, expert of c].
// Columns below E * ff belong to expert c / ff and take `limit`; the columns beyond belong to one more expert (index E)
// with `limit_rest`. weights null: no scaling.
template <typename TH>
__global__ void __launch_bounds__(256)
expert_act_kernel(const float* __restrict__ z, int ldz, int total, TH* __restrict__ hidden, const float* __restrict__ weights,
                  int ldw, int T, int E, int ff, float limit, float limit_rest, float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long n = (long long)T * total;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / total;
        const int c = (int)(i - t * total);
        const int e = c < E * ff ? c / ff : E;
        const float lim = e < E ? limit : limit_rest;
        const float g = fminf(z[t * ldz + c], lim);
        const float u = fminf(fmaxf(z[t * ldz + total + c], -lim), lim);
        float v = g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
        if (weights) v *= weights[t * ldw + e];
        hidden[i] = lp_from_float<TH>(v);
    }
}

// The same, four columns of one expert per thread and a token per blockIdx.y (expert sizes, row lengths and strides of a
// multiple of four values, bfloat16 out): two float4 loads, one 8-byte store.
__global__ void __launch_bounds__(256)
expert_act_vec4_kernel(const float* __restrict__ z, int ldz, int total, __nv_bfloat16* __restrict__ hidden,
                       const float* __restrict__ weights, int ldw, int E, int ff, float limit, float limit_rest,
                       float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long t = blockIdx.y;
    const float* row = z + t * ldz;
    const int quads = total / 4;
    for (int q = blockIdx.x * blockDim.x + threadIdx.x; q < quads; q += gridDim.x * blockDim.x) {
        const int c = q * 4;
        const int e = c < E * ff ? c / ff : E;
        const float lim = e < E ? limit : limit_rest;
        const float w = weights ? weights[t * ldw + e] : 1.0f;
        const float4 g4 = *reinterpret_cast<const float4*>(row + c);
        const float4 u4 = *reinterpret_cast<const float4*>(row + total + c);
        const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float g = fminf(gs[k], lim);
            const float u = fminf(fmaxf(us[k], -lim), lim);
            v[k] = g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
            if (weights) v[k] *= w;
        }
        uint2 packed;
        *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(hidden + t * total + c) = packed;
    }
}


// A third rule: scores s = softmax(z) over all E router outputs. The choice is made on s[e] + correction[e]: the
// experts form `groups` equal groups of neighbours, a group's score is its largest choice score, only experts of the
// `keep` best groups may be chosen (the others count as minus infinity: choice scores may be negative), and the `top`
// largest choice scores among those win. The weights are the chosen experts' scores s themselves (without the
// correction) times `scale`; they are not renormalised. A warp per token; among equal scores the lower index wins.
__global__ void __launch_bounds__(128)
route_softmax_kernel(const float* __restrict__ z, int ldz, const float* __restrict__ correction, float* __restrict__ weights,
                     int ldw, int T, int E, int groups, int keep, int top, float scale) {
    extern __shared__ float sm[];
    lp_grid_release();
    lp_grid_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = sm + (size_t)warp * (3 * E + groups);
    float* choice = s + E;
    float* flag = choice + E;
    float* gs = flag + E;
    const int per = E / groups;
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[t * ldz + e]);
    mx = lp_warp_max(mx);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(z[t * ldz + e] - mx);
        s[e] = v;
        sum += v;
    }
    sum = lp_warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) {
        const float v = s[e] * inv;
        s[e] = v;
        choice[e] = v + (correction ? correction[e] : 0.f);
        flag[e] = groups > 1 ? 0.f : 1.f;
    }
    __syncwarp();
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY;
            for (int j = 0; j < per; ++j) a = fmaxf(a, choice[g * per + j]);
            gs[g] = a;
        }
        __syncwarp();
        if (lane == 0) {
            for (int n = 0; n < keep; ++n) {
                int best = -1;
                float bv = -INFINITY;
                for (int g = 0; g < groups; ++g)
                    if (gs[g] > bv) { bv = gs[g]; best = g; }
                if (best < 0) break;
                gs[best] = -INFINITY;
                for (int j = 0; j < per; ++j) flag[best * per + j] = 1.f;
            }
        }
        __syncwarp();
    }
    if (lane == 0) {
        for (int n = 0; n < top; ++n) {
            int best = -1;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (flag[e] == 1.f && choice[e] > bv) { bv = choice[e]; best = e; }
            if (best < 0) break;
            flag[best] = 2.f;
        }
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) weights[t * ldw + e] = flag[e] == 2.f ? s[e] * scale : 0.f;
}

// x[t, :] += h[t, :] * sum_{e in [first, first + count)} weights[t, e]: experts that are the identity pass the
// feed-forward's input on, times their weight. x float32 [T, d]; h [T, d] in the activations' format.
template <typename TH>
__global__ void __launch_bounds__(256)
identity_experts_kernel(float* __restrict__ x, const TH* __restrict__ h, const float* __restrict__ weights, int ldw, int first,
                        int count, int T, int d) {
    lp_grid_release();
    lp_grid_wait();
    const long long n = (long long)T * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / d;
        float w = 0.f;
        for (int e = 0; e < count; ++e) w += weights[t * ldw + first + e];
        if (w != 0.f) x[i] = fmaf(lp_to_float(h[i]), w, x[i]);
    }
}

}  // namespace

// z: float32 [T, ldz] (E logits per row); weights: float32 [T, ldw], E values per row written.
extern "C" int lp_route(const float* z, int ldz, float* weights, int ldw, int T, int E, int groups, int keep, int top,
                        cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || groups <= 0 || E % groups) LP_REFUSE("route: %d experts in %d groups", E, groups);
    if (keep <= 0 || keep > groups) LP_REFUSE("route: %d of %d groups kept", keep, groups);
    if (top <= 0 || top > keep * (E / groups)) LP_REFUSE("route: %d experts chosen from %d groups of %d", top, keep, E / groups);
    if (ldz < E || ldw < E) LP_REFUSE("route: rows of %d and %d values for %d experts", ldz, ldw, E);
    const size_t smem = (size_t)4 * (2 * E + groups) * sizeof(float);
    if (smem > 48 * 1024) LP_REFUSE("route: %d experts need %zu bytes of shared memory", E, smem);
    lp_launch(route_kernel, (unsigned)((T + 3) / 4), 128, smem, stream, z, ldz, weights, ldw, T, E, groups, keep, top);
    return lp_check_launch("route");
}

// zero (optional): a float32 buffer of zero_count values cleared on the side, for the product after the scaling when it
// sums partial results into its output.
// id_x (optional): float32 [T, d], to which h [T, d] (dtype code id_dtype) times the sum of the weights' columns
// id_first .. id_first + id_count - 1 is added in the same launch (experts that pass their input on).
extern "C" int lp_expert_scale(void* hidden, int dtype, int ldh, const float* weights, int ldw, int T, int E, int ff,
                               float* zero, long long zero_count, float* id_x, const void* id_h, int id_dtype, int id_first,
                               int id_count, int id_d, cudaStream_t stream) {
    if (T <= 0 || E <= 0 || ff <= 0) return 0;
    IdentityShare id{};
    if (id_x && id_count > 0) {
        if (!id_h || id_d <= 0 || id_first < 0 || id_first + id_count > ldw || (id_dtype != LP_F32 && id_dtype != LP_BF16))
            LP_REFUSE("expert_scale: identity columns %d..%d of rows of %d, width %d, dtype code %d", id_first, id_first + id_count - 1, ldw, id_d, id_dtype);
        id = IdentityShare{id_x, id_h, id_dtype == LP_BF16 ? 1 : 0, id_first, id_count, id_d};
    }
    if (ldh < E * ff || ldw < E) LP_REFUSE("expert_scale: rows of %d and %d values for %d experts of %d", ldh, ldw, E, ff);
    const long long n = (long long)T * E * ff;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == LP_BF16 && ff % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)hidden & 15) == 0 && T <= 65535) {
        const int octets = E * ff / 8;
        int bx = (octets + 255) / 256;
        if (bx > 64) bx = 64;
        lp_launch(expert_scale_vec8_kernel, dim3(bx, T), 256, 0, stream, (__nv_bfloat16*)hidden, ldh, weights, ldw, E, ff, zero, zero_count, id);
        return lp_check_launch("expert_scale");
    }
    if (dtype == LP_F32) lp_launch(expert_scale_kernel<float>, (unsigned)blocks, 256, 0, stream, (float*)hidden, ldh, weights, ldw, T, E, ff, zero, zero_count, id);
    else if (dtype == LP_BF16) lp_launch(expert_scale_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, (__nv_bfloat16*)hidden, ldh, weights, ldw, T, E, ff, zero, zero_count, id);
    else LP_REFUSE("expert_scale: dtype code %d", dtype);
    return lp_check_launch("expert_scale");
}

// z: float32 [T, ldz] (E logits per row, then `extra` gate columns); bias: float32 [E] or null; weights: float32
// [T, ldw], E + extra values per row written.
extern "C" int lp_route_top(const float* z, int ldz, const float* bias, float* weights, int ldw, int T, int E, int top,
                            int extra, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || extra < 0) LP_REFUSE("route_top: %d of %d experts, %d gates", top, E, extra);
    if (ldz < E + extra || ldw < E + extra) LP_REFUSE("route_top: rows of %d and %d values for %d columns", ldz, ldw, E + extra);
    const size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 48 * 1024) LP_REFUSE("route_top: %d experts need %zu bytes of shared memory", E, smem);
    lp_launch(route_top_kernel, (unsigned)((T + 3) / 4), 128, smem, stream, z, ldz, bias, weights, ldw, T, E, top, extra);
    return lp_check_launch("route_top");
}

// z: float32 [T, ldz] with the gate sums of `total` hidden columns, then their up sums; hidden: [T, total].
extern "C" int lp_expert_act(const float* z, int ldz, int total, void* hidden, int dtype, const float* weights, int ldw,
                             int T, int E, int ff, float limit, float limit_rest, float* zero, long long zero_count,
                             cudaStream_t stream) {
    if (T <= 0 || total <= 0) return 0;
    if (E < 0 || ff <= 0 || (long long)E * ff > total) LP_REFUSE("expert_act: %d experts of %d in %d columns", E, ff, total);
    if (ldz < 2 * total) LP_REFUSE("expert_act: rows of %d values for 2 x %d sums", ldz, total);
    if (weights && ldw < E + (total > E * ff ? 1 : 0)) LP_REFUSE("expert_act: rows of %d weights", ldw);
    const long long n = (long long)T * total;
    if (dtype == LP_BF16 && total % 4 == 0 && ff % 4 == 0 && ldz % 4 == 0 && T <= 65535 &&
        (reinterpret_cast<uintptr_t>(z) & 15) == 0 && (reinterpret_cast<uintptr_t>(hidden) & 7) == 0) {
        int bx = (total / 4 + 255) / 256;
        if (bx > 32) bx = 32;
        lp_launch(expert_act_vec4_kernel, dim3(bx, T), 256, 0, stream, z, ldz, total, (__nv_bfloat16*)hidden, weights, ldw, E, ff,
                  limit, limit_rest, zero, zero_count);
        return lp_check_launch("expert_act");
    }
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == LP_F32) lp_launch(expert_act_kernel<float>, (unsigned)blocks, 256, 0, stream, z, ldz, total, (float*)hidden, weights, ldw, T, E, ff, limit, limit_rest, zero, zero_count);
    else if (dtype == LP_BF16) lp_launch(expert_act_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, z, ldz, total, (__nv_bfloat16*)hidden, weights, ldw, T, E, ff, limit, limit_rest, zero, zero_count);
    else LP_REFUSE("expert_act: dtype code %d", dtype);
    return lp_check_launch("expert_act");
}

// z: float32 [T, ldz], E router outputs per row; correction: float32 [E] or null; weights: float32 [T, ldw].
extern "C" int lp_route_softmax(const float* z, int ldz, const float* correction, float* weights, int ldw, int T, int E,
                                int groups, int keep, int top, float scale, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (E <= 0 || groups <= 0 || E % groups) LP_REFUSE("route_softmax: %d experts in %d groups", E, groups);
    if (keep <= 0 || keep > groups) LP_REFUSE("route_softmax: %d of %d groups kept", keep, groups);
    if (top <= 0 || top > keep * (E / groups)) LP_REFUSE("route_softmax: %d experts chosen from %d groups of %d", top, keep, E / groups);
    if (ldz < E || ldw < E) LP_REFUSE("route_softmax: rows of %d and %d values for %d experts", ldz, ldw, E);
    const size_t smem = (size_t)4 * (3 * E + groups) * sizeof(float);
    if (smem > 48 * 1024) LP_REFUSE("route_softmax: %d experts need %zu bytes of shared memory", E, smem);
    lp_launch(route_softmax_kernel, (unsigned)((T + 3) / 4), 128, smem, stream, z, ldz, correction, weights, ldw, T, E, groups,
              keep, top, scale);
    return lp_check_launch("route_softmax");
}

// x: float32 [T, d]; h: [T, d] (dtype code); weights: float32 [T, ldw]; columns first .. first + count - 1 are summed.
extern "C" int lp_identity_experts(float* x, const void* h, int dtype, const float* weights, int ldw, int first, int count,
                                   int T, int d, cudaStream_t stream) {
    if (T <= 0 || d <= 0 || count <= 0) return 0;
    if (first < 0 || first + count > ldw) LP_REFUSE("identity_experts: columns %d..%d of rows of %d", first, first + count - 1, ldw);
    long long blocks = ((long long)T * d + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == LP_F32) lp_launch(identity_experts_kernel<float>, (unsigned)blocks, 256, 0, stream, x, (const float*)h, weights, ldw, first, count, T, d);
    else if (dtype == LP_BF16) lp_launch(identity_experts_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, x, (const __nv_bfloat16*)h, weights, ldw, first, count, T, d);
    else LP_REFUSE("identity_experts: dtype code %d", dtype);
    return lp_check_launch("identity_experts");
}
