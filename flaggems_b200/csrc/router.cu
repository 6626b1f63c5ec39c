// Router kernels in front of the fused MoE path: softmax + top-k, and group-limited top-k
// (DeepSeek-V3 routing).  One warp per token: the expert scores of a row live in registers
// (topk_softmax) or in the warp's slice of shared memory (grouped_topk), every reduction is a
// shuffle tree, ties go to the lower index.  Both kernels can also count how many route slots
// each expert received (the histogram the expert-parallel dispatch plan starts from).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int WARPS_PER_CTA = 4;
#define NEG_INF (-INFINITY)

__device__ __forceinline__ float load_score(const void* p, int dtype, int64_t i) {
    if (dtype == FG_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    if (dtype == FG_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float round_to(float v, int dtype) {
    if (dtype == FG_DTYPE_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (dtype == FG_DTYPE_F16) return __half2float(__float2half_rn(v));
    return v;
}

// (value, index) arg-max over the warp: larger value wins, equal values go to the lower index.
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, off);
        const int oi = __shfl_xor_sync(0xffffffffu, i, off);
        if (ov > v || (ov == v && oi < i)) {
            v = ov;
            i = oi;
        }
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ void store_index(void* p, int index_kind, int64_t at, int v) {
    if (index_kind == 2) reinterpret_cast<int64_t*>(p)[at] = (int64_t)v;
    else reinterpret_cast<int32_t*>(p)[at] = v;  // int32 and uint32 share the bit pattern
}

struct TopkSoftmaxArgs {
    const void* gating;
    int gating_dtype;
    float* weights;
    void* indices;
    int index_kind;
    int32_t* source_rows;
    int32_t* expert_counts;
    int64_t T;
    int E, k, renormalize;
};

// VPT values per lane; expert e = lane + 32 * j.
template <int VPT>
__global__ void __launch_bounds__(32 * WARPS_PER_CTA) topk_softmax_kernel(const TopkSoftmaxArgs a) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * WARPS_PER_CTA + (threadIdx.x >> 5);
    if (row >= a.T) return;
    float p[VPT];
    float mx = NEG_INF;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int e = lane + 32 * j;
        p[j] = e < a.E ? load_score(a.gating, a.gating_dtype, row * a.E + e) : NEG_INF;
        mx = fmaxf(mx, p[j]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        p[j] = expf(p[j] - mx);  // exp(-inf) = 0 for the padding
        sum += p[j];
    }
    sum = warp_sum(sum) + 1e-8f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) p[j] = (lane + 32 * j < a.E) ? p[j] / sum : NEG_INF;

    float my_w = 0.0f;  // lane ki keeps the weight of round ki
    int my_i = 0;
    float selected_sum = 0.0f;
    for (int ki = 0; ki < a.k; ++ki) {
        float v = NEG_INF;
        int idx = lane;
#pragma unroll
        for (int j = 0; j < VPT; ++j)
            if (p[j] > v) {
                v = p[j];
                idx = lane + 32 * j;
            }
        warp_argmax(v, idx);
        if (lane == ki) {
            my_w = v;
            my_i = idx;
        }
        selected_sum += v;
        if ((idx & 31) == lane) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
                if (j == (idx >> 5)) p[j] = NEG_INF;
        }
    }
    if (lane < a.k) {
        if (a.renormalize) my_w = my_w / (selected_sum + 1e-8f);
        const int64_t at = row * a.k + lane;
        a.weights[at] = my_w;
        store_index(a.indices, a.index_kind, at, my_i);
        a.source_rows[at] = (int32_t)((int64_t)lane * a.T + row);
        if (a.expert_counts) atomicAdd(&a.expert_counts[my_i], 1);
    }
}

struct GroupedTopkArgs {
    const void* scores;
    const void* bias;
    int dtype;
    float* values;
    int32_t* indices;
    int32_t* expert_counts;
    int64_t T, stride;
    int E, n_group, topk_group, topk, renormalize, sigmoid;
    float scaling;
};

__device__ __forceinline__ float processed_score(const GroupedTopkArgs& a, int64_t row, int e) {
    float s = load_score(a.scores, a.dtype, row * a.stride + e);
    if (a.sigmoid) s = round_to(__fdiv_rn(1.0f, 1.0f + expf(-s)), a.dtype);
    return s;
}

__global__ void __launch_bounds__(32 * WARPS_PER_CTA) grouped_topk_kernel(const GroupedTopkArgs a) {
    extern __shared__ float smem_scores[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t row = (int64_t)blockIdx.x * WARPS_PER_CTA + warp;
    if (row >= a.T) return;
    float* xb = smem_scores + (size_t)warp * a.E;  // (score + bias), added in the input dtype
    for (int e = lane; e < a.E; e += 32)
        xb[e] = round_to(processed_score(a, row, e) + load_score(a.bias, a.dtype, e), a.dtype);
    __syncwarp();

    // Score of each group = its two largest entries added (the maximum twice when it repeats).
    const int epg = a.E / a.n_group;
    float my_group = NEG_INF;  // lane g keeps group g
    for (int g = 0; g < a.n_group; ++g) {
        const float* x = xb + g * epg;
        float m1 = NEG_INF;
        for (int e = lane; e < epg; e += 32) m1 = fmaxf(m1, x[e]);
        m1 = warp_max(m1);
        int cnt = 0;
        for (int e = lane; e < epg; e += 32) cnt += (x[e] == m1) ? 1 : 0;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, off);
        float m2 = NEG_INF;
        for (int e = lane; e < epg; e += 32) {
            const float v = x[e];
            m2 = fmaxf(m2, (v == m1 && cnt == 1) ? NEG_INF : v);
        }
        m2 = warp_max(m2);
        float gs = round_to(m1 + m2, a.dtype);
        if (!(gs == gs) || gs == INFINITY) gs = NEG_INF;  // NaN and +inf do not compete
        if (lane == g) my_group = gs;
    }
    const bool proceed = warp_max(my_group) != NEG_INF;

    // The topk_group best groups; equal scores go to the lower group index.
    int rank = 0;
    for (int j = 0; j < a.n_group; ++j) {
        const float other = __shfl_sync(0xffffffffu, my_group, j);
        rank += (other > my_group || (other == my_group && j < lane)) ? 1 : 0;
    }
    const unsigned chosen = __ballot_sync(0xffffffffu, lane < a.n_group && rank < a.topk_group);
    for (int e = lane; e < a.E; e += 32)
        if (!((chosen >> (e / epg)) & 1u)) xb[e] = NEG_INF;
    __syncwarp();

    float my_v = 0.0f;
    int my_i = 0;
    for (int ki = 0; ki < a.topk; ++ki) {
        float v = NEG_INF;
        int idx = lane;  // lowest index this lane owns, should all of its entries be -inf
        for (int e = lane; e < a.E; e += 32)
            if (xb[e] > v) {
                v = xb[e];
                idx = e;
            }
        warp_argmax(v, idx);
        if (lane == ki) {
            my_i = idx;
            my_v = processed_score(a, row, idx);  // the weight is the score without the bias
        }
        if ((idx & 31) == lane) xb[idx] = NEG_INF;
        __syncwarp();
    }
    const float total = warp_sum(lane < a.topk ? my_v : 0.0f);
    const float scale = a.renormalize ? a.scaling / (total + 1e-20f) : a.scaling;
    if (lane < a.topk) {
        const int64_t at = row * a.topk + lane;
        const float v = proceed ? my_v * scale : 1.0f / (float)a.topk;
        const int i = proceed ? my_i : lane;
        a.values[at] = v;
        a.indices[at] = i;
        if (a.expert_counts) atomicAdd(&a.expert_counts[i], 1);
    }
}

bool score_dtype_ok(int d) { return d == FG_DTYPE_BF16 || d == FG_DTYPE_F16 || d == FG_DTYPE_F32; }

}  // namespace

extern "C" {

int fg_topk_softmax(float* topk_weights, void* topk_indices, int index_kind, int32_t* token_expert_indices,
                    const void* gating_output, int gating_dtype, int64_t num_tokens, int num_experts, int topk,
                    int renormalize, int32_t* expert_counts, void* stream) {
    FG_REQUIRE(num_tokens >= 0 && num_experts > 0 && topk > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(topk <= 32, FG_ERR_INVALID_ARGUMENT, "topk %d must be at most 32", topk);
    FG_REQUIRE(num_experts <= 1024, FG_ERR_UNSUPPORTED, "num_experts %d must be at most 1024", num_experts);
    FG_REQUIRE(index_kind >= 0 && index_kind <= 2, FG_ERR_INVALID_ARGUMENT, "topk_indices must be int32/int64/uint32");
    FG_REQUIRE(score_dtype_ok(gating_dtype), FG_ERR_INVALID_ARGUMENT, "bad gating dtype %d", gating_dtype);
    if (num_tokens == 0) return FG_OK;
    FG_REQUIRE(topk_weights && topk_indices && token_expert_indices && gating_output, FG_ERR_INVALID_ARGUMENT,
               "null pointer");
    FG_REQUIRE(num_tokens * topk < (1ll << 31), FG_ERR_UNSUPPORTED, "too many route slots");
    TopkSoftmaxArgs a{gating_output, gating_dtype, topk_weights, topk_indices, index_kind, token_expert_indices,
                      expert_counts, num_tokens, num_experts, topk, renormalize};
    const unsigned grid = (unsigned)fg_cdiv(num_tokens, WARPS_PER_CTA);
    const int threads = 32 * WARPS_PER_CTA;
    cudaStream_t st = (cudaStream_t)stream;
    const int vpt = (num_experts + 31) / 32;
    if (vpt <= 1) topk_softmax_kernel<1><<<grid, threads, 0, st>>>(a);
    else if (vpt <= 2) topk_softmax_kernel<2><<<grid, threads, 0, st>>>(a);
    else if (vpt <= 4) topk_softmax_kernel<4><<<grid, threads, 0, st>>>(a);
    else if (vpt <= 8) topk_softmax_kernel<8><<<grid, threads, 0, st>>>(a);
    else if (vpt <= 16) topk_softmax_kernel<16><<<grid, threads, 0, st>>>(a);
    else topk_softmax_kernel<32><<<grid, threads, 0, st>>>(a);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_grouped_topk(float* topk_values, int32_t* topk_indices, const void* scores, const void* bias, int dtype,
                    int64_t num_tokens, int num_experts, int64_t scores_stride, int n_group, int topk_group, int topk,
                    int renormalize, float routed_scaling_factor, int scoring_func, int32_t* expert_counts,
                    void* stream) {
    FG_REQUIRE(num_tokens >= 0 && num_experts > 0 && n_group > 0 && topk > 0 && topk_group > 0,
               FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(num_experts % n_group == 0, FG_ERR_INVALID_ARGUMENT, "num_experts must be divisible by n_group");
    FG_REQUIRE(n_group <= 32, FG_ERR_INVALID_ARGUMENT, "n_group should be smaller than or equal to 32");
    FG_REQUIRE(topk <= 32, FG_ERR_INVALID_ARGUMENT, "topk should be smaller than or equal to 32 for now");
    FG_REQUIRE(scoring_func == 0 || scoring_func == 1, FG_ERR_INVALID_ARGUMENT,
               "scoring_func must be 0 (none) or 1 (sigmoid)");
    FG_REQUIRE(score_dtype_ok(dtype), FG_ERR_INVALID_ARGUMENT, "Unsupported dtype: %d", dtype);
    FG_REQUIRE(num_experts <= 2048, FG_ERR_UNSUPPORTED, "num_experts %d must be at most 2048", num_experts);
    FG_REQUIRE(scores_stride >= num_experts, FG_ERR_INVALID_ARGUMENT, "row stride smaller than num_experts");
    if (num_tokens == 0) return FG_OK;
    FG_REQUIRE(topk_values && topk_indices && scores && bias, FG_ERR_INVALID_ARGUMENT, "null pointer");
    GroupedTopkArgs a{scores, bias, dtype, topk_values, topk_indices, expert_counts, num_tokens, scores_stride,
                      num_experts, n_group, topk_group, topk, renormalize, scoring_func, routed_scaling_factor};
    const unsigned grid = (unsigned)fg_cdiv(num_tokens, WARPS_PER_CTA);
    const size_t smem = (size_t)WARPS_PER_CTA * num_experts * sizeof(float);
    grouped_topk_kernel<<<grid, 32 * WARPS_PER_CTA, smem, (cudaStream_t)stream>>>(a);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

}  // extern "C"
