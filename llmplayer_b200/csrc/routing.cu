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
template <typename TH>
__global__ void __launch_bounds__(256)
expert_scale_kernel(TH* __restrict__ hidden, int ldh, const float* __restrict__ weights, int ldw, int T, int E, int ff,
                    float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
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
                         float* __restrict__ zero, long long zero_count) {
    lp_grid_release();
    lp_grid_wait();
    clear_on_the_side(zero, zero_count);
    const long long t = blockIdx.y;
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
extern "C" int lp_expert_scale(void* hidden, int dtype, int ldh, const float* weights, int ldw, int T, int E, int ff,
                               float* zero, long long zero_count, cudaStream_t stream) {
    if (T <= 0 || E <= 0 || ff <= 0) return 0;
    if (ldh < E * ff || ldw < E) LP_REFUSE("expert_scale: rows of %d and %d values for %d experts of %d", ldh, ldw, E, ff);
    const long long n = (long long)T * E * ff;
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == LP_BF16 && ff % 8 == 0 && ldh % 8 == 0 && ((uintptr_t)hidden & 15) == 0 && T <= 65535) {
        const int octets = E * ff / 8;
        int bx = (octets + 255) / 256;
        if (bx > 64) bx = 64;
        lp_launch(expert_scale_vec8_kernel, dim3(bx, T), 256, 0, stream, (__nv_bfloat16*)hidden, ldh, weights, ldw, E, ff, zero, zero_count);
        return lp_check_launch("expert_scale");
    }
    if (dtype == LP_F32) lp_launch(expert_scale_kernel<float>, (unsigned)blocks, 256, 0, stream, (float*)hidden, ldh, weights, ldw, T, E, ff, zero, zero_count);
    else if (dtype == LP_BF16) lp_launch(expert_scale_kernel<__nv_bfloat16>, (unsigned)blocks, 256, 0, stream, (__nv_bfloat16*)hidden, ldh, weights, ldw, T, E, ff, zero, zero_count);
    else LP_REFUSE("expert_scale: dtype code %d", dtype);
    return lp_check_launch("expert_scale");
}
