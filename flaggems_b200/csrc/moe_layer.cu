// Routed-expert pipeline of the block-FP8 MoE layer as ONE host call: align -> gather (and
// quantise) into expert-sorted padded order -> grouped GEMM1 with fused SiLU*up -> group
// quantisation -> grouped GEMM2 with the router weight.  Five launches issued back to back from
// C++, so the host cost of a layer step does not grow with the number of kernels.  All scratch
// lives in a caller-provided workspace; nothing is allocated here.
#include <mutex>

#include "common.cuh"

// Built-in scratch of fg_moe_routed_block_fp8_local_noalloc: part of the library image, so every
// GPU on which the library is loaded keeps these bytes reserved until the process exits.
// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_routed_scratch[FG_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int TILE_ROWS = 128;

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

struct Workspace {
    int32_t* sorted_ids;
    int32_t* expert_ids;
    int32_t* post_pad;
    uint8_t* a1;
    float* a1s;
    uint8_t* act;
    uint8_t* a2;
    float* a2s;
    int64_t max_pad, n_blocks, rows, bytes;
};

Workspace carve(void* base, int64_t n_in, int num_experts, int64_t H, int64_t I, int out_esz) {
    Workspace w{};
    w.max_pad = n_in + (int64_t)num_experts * (TILE_ROWS - 1);
    w.n_blocks = fg_cdiv(w.max_pad, TILE_ROWS);
    w.rows = w.max_pad / TILE_ROWS * TILE_ROWS;
    uint8_t* p = reinterpret_cast<uint8_t*>(base);
    int64_t off = 0;
    auto take = [&](int64_t bytes) {
        uint8_t* r = p ? p + off : nullptr;
        off += align_up(bytes, 256);
        return r;
    };
    w.sorted_ids = (int32_t*)take(4 * w.max_pad);
    w.expert_ids = (int32_t*)take(4 * w.n_blocks);
    w.post_pad = (int32_t*)take(256);
    w.a1 = take(w.rows * H);
    w.a1s = (float*)take(4 * w.rows * (H / 128));
    w.act = take(w.rows * I * out_esz);
    w.a2 = take(w.rows * I);
    w.a2s = (float*)take(4 * w.rows * (I / 128));
    w.bytes = off;
    return w;
}

int check_dims(int64_t n_in, int num_experts, int64_t H, int64_t I, int out_dtype) {
    FG_REQUIRE(n_in >= 0 && num_experts > 0 && H > 0 && I > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(H % 128 == 0 && I % 128 == 0, FG_ERR_UNSUPPORTED,
               "hidden %lld and intermediate %lld must be multiples of 128", (long long)H, (long long)I);
    FG_REQUIRE(out_dtype == FG_DTYPE_BF16 || out_dtype == FG_DTYPE_F16, FG_ERR_UNSUPPORTED,
               "activations must be bf16 or fp16");
    return FG_OK;
}

// GEMM1 -> quant -> GEMM2 on rows already in sorted order in ws.a1 / ws.a1s.
int run_gemms(void* y, const Workspace& ws, int64_t n_in, const void* w1, const void* w2, const float* s1,
              const float* s2, int num_experts, int64_t H, int64_t I, const void* weights, int w_dtype,
              int64_t w_stride, int out_dtype, const int32_t* dest, int64_t dest_stride, void* const* peer_out,
              int n_peers, int64_t peer_rows, void* stream) {
    int rc = fg_moe_grouped_gemm_fp8(ws.act, ws.a1, w1, ws.a1s, s1, nullptr, 0, 1, ws.sorted_ids, ws.expert_ids,
                                     ws.post_pad, ws.rows, n_in, num_experts, 2 * I, H, H, I, TILE_ROWS, FG_SCALE_BLOCK,
                                     1, /*fuse_silu=*/1, /*scatter=*/0, /*mul_weight=*/0, out_dtype, stream);
    if (rc != FG_OK) return rc;
    rc = fg_per_token_group_quant_fp8_gather(ws.act, out_dtype, ws.a2, ws.a2s, ws.rows, I, 128, I, I, nullptr, 1, 0,
                                             ws.post_pad, stream);
    if (rc != FG_OK) return rc;
    return fg_moe_grouped_gemm_fp8_peer(y, ws.a2, w2, ws.a2s, s2, weights, w_dtype, w_stride, ws.sorted_ids,
                                        ws.expert_ids, ws.post_pad, ws.rows, n_in, num_experts, H, I, I, H, TILE_ROWS,
                                        FG_SCALE_BLOCK, 1, /*fuse_silu=*/0, /*scatter=*/1, /*mul_weight=*/1, out_dtype,
                                        dest, dest_stride, peer_out, n_peers, peer_rows, stream);
}

// Device address of g_routed_scratch on the current device, looked up once per device.
int builtin_scratch(void** out) {
    static std::mutex mu;
    static void* addr[64] = {nullptr};
    int dev = -1;
    FG_CUDA(cudaGetDevice(&dev));
    FG_REQUIRE(dev >= 0 && dev < 64, FG_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void* p = nullptr;
        FG_CUDA(cudaGetSymbolAddress((void**)&p, g_routed_scratch));
        addr[dev] = p;
    }
    *out = addr[dev];
    return FG_OK;
}

}  // namespace

namespace {

// Scratch of fg_scaled_grouped_mm_fp8.
struct GroupedMmWorkspace {
    int32_t* group_ids;
    int32_t* sorted_ids;
    int32_t* expert_ids;
    int32_t* post_pad;
    uint8_t* a_sorted;
    float* sa_sorted;
    int64_t max_pad, n_blocks, rows, bytes;
};

GroupedMmWorkspace carve_grouped_mm(void* base, int64_t m_total, int num_groups, int64_t K) {
    GroupedMmWorkspace w{};
    w.max_pad = m_total + (int64_t)num_groups * (TILE_ROWS - 1);
    w.n_blocks = fg_cdiv(w.max_pad, TILE_ROWS);
    w.rows = w.max_pad / TILE_ROWS * TILE_ROWS;
    uint8_t* p = reinterpret_cast<uint8_t*>(base);
    int64_t off = 0;
    auto take = [&](int64_t bytes) {
        uint8_t* r = p ? p + off : nullptr;
        off += align_up(bytes, 256);
        return r;
    };
    w.group_ids = (int32_t*)take(4 * m_total);
    w.sorted_ids = (int32_t*)take(4 * w.max_pad);
    w.expert_ids = (int32_t*)take(4 * w.n_blocks);
    w.post_pad = (int32_t*)take(256);
    w.a_sorted = take(w.rows * K);
    w.sa_sorted = (float*)take(4 * w.rows);
    w.bytes = off;
    return w;
}

}  // namespace

extern "C" {

int64_t fg_scaled_grouped_mm_workspace_bytes(int64_t m_total, int num_groups, int64_t K) {
    if (m_total < 0 || num_groups <= 0 || K <= 0) return -1;
    return carve_grouped_mm(nullptr, m_total, num_groups, K).bytes;
}

int fg_scaled_grouped_mm_fp8(void* c, const void* a, const void* b, const float* scale_a, const float* scale_b,
                             const float* bias, int64_t bias_stride_g, const int32_t* offs, int num_groups,
                             int64_t m_total, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c, int out_dtype,
                             void* workspace, int64_t workspace_bytes, void* stream) {
    FG_REQUIRE(m_total >= 0 && N > 0 && K > 0 && num_groups > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(num_groups <= 1024, FG_ERR_UNSUPPORTED, "at most 1024 groups");
    FG_REQUIRE(K % 16 == 0, FG_ERR_UNSUPPORTED, "K = %lld must be a multiple of 16", (long long)K);
    if (m_total == 0) return FG_OK;
    FG_REQUIRE(c && a && b && scale_a && scale_b && offs && workspace, FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE((uintptr_t)workspace % 256 == 0, FG_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    const GroupedMmWorkspace ws = carve_grouped_mm(workspace, m_total, num_groups, K);
    FG_REQUIRE(workspace_bytes >= ws.bytes, FG_ERR_INVALID_ARGUMENT, "workspace holds %lld bytes, needs %lld",
               (long long)workspace_bytes, (long long)ws.bytes);
    int rc = fg_group_ids_from_offsets(offs, num_groups, m_total, ws.group_ids, stream);
    if (rc != FG_OK) return rc;
    rc = fg_moe_align_block_size(ws.group_ids, 0, m_total, num_groups, TILE_ROWS, nullptr, 0, ws.sorted_ids, ws.max_pad,
                                 ws.expert_ids, ws.n_blocks, ws.post_pad, stream);
    if (rc != FG_OK) return rc;
    rc = fg_gather_rows_fp8(a, scale_a, ws.a_sorted, ws.sa_sorted, ws.rows, K, 1, ld_a, 1, ws.sorted_ids, 1,
                            (int32_t)m_total, ws.post_pad, stream);
    if (rc != FG_OK) return rc;
    return fg_grouped_gemm_fp8_bias(c, ws.a_sorted, b, ws.sa_sorted, scale_b, bias, bias_stride_g, ws.sorted_ids,
                                    ws.expert_ids, ws.post_pad, ws.rows, m_total, num_groups, N, K, K, ld_c, out_dtype,
                                    stream);
}

int64_t fg_moe_routed_workspace_bytes(int64_t n_rows_in, int num_experts, int64_t H, int64_t I) {
    if (n_rows_in < 0 || num_experts <= 0 || H <= 0 || I <= 0) return -1;
    return carve(nullptr, n_rows_in, num_experts, H, I, 2).bytes;
}

int fg_moe_routed_block_fp8_local(void* y, const void* hidden, int hidden_dtype, const void* topk_ids,
                                  int ids_are_i64, const void* topk_w, int topk_w_dtype, int64_t T, int topk,
                                  const void* w1, const void* w2, const float* s1, const float* s2, int num_experts,
                                  int64_t H, int64_t I, void* workspace, int64_t workspace_bytes, void* stream) {
    const int64_t n_in = T * topk;
    int rc = check_dims(n_in, num_experts, H, I, hidden_dtype);
    if (rc != FG_OK) return rc;
    if (n_in == 0) return FG_OK;
    FG_REQUIRE(y && hidden && topk_ids && topk_w && w1 && w2 && s1 && s2 && workspace, FG_ERR_INVALID_ARGUMENT,
               "null pointer");
    FG_REQUIRE((uintptr_t)workspace % 256 == 0, FG_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    const Workspace ws = carve(workspace, n_in, num_experts, H, I, 2);
    FG_REQUIRE(workspace_bytes >= ws.bytes, FG_ERR_INVALID_ARGUMENT, "workspace holds %lld bytes, needs %lld",
               (long long)workspace_bytes, (long long)ws.bytes);
    rc = fg_moe_align_block_size(topk_ids, ids_are_i64, n_in, num_experts, TILE_ROWS, nullptr, 0, ws.sorted_ids,
                                 ws.max_pad, ws.expert_ids, ws.n_blocks, ws.post_pad, stream);
    if (rc != FG_OK) return rc;
    // Every token is quantised once (as the reference does before its gathering GEMM) and its FP8 row
    // and scales are then copied to each of its top-k places in expert order: quantising while gathering
    // would read and quantise every token top-k times.  The token buffer borrows the room of GEMM1's
    // output, which is first written after the copy has finished.  Bits are the same either way.
    const int64_t s_cols = H / 128;
    const int64_t tok_q_bytes = align_up(T * H, 256);
    if (topk > 1 && tok_q_bytes + 4 * T * s_cols <= ws.rows * I * 2) {
        uint8_t* tok_q = ws.act;
        float* tok_s = reinterpret_cast<float*>(ws.act + tok_q_bytes);
        rc = fg_per_token_group_quant_fp8(hidden, hidden_dtype, tok_q, tok_s, T, H, 128, H, H, s_cols, 1, 1e-10f, 0,
                                          stream);
        if (rc != FG_OK) return rc;
        rc = fg_gather_rows_fp8(tok_q, tok_s, ws.a1, ws.a1s, ws.rows, H, s_cols, H, s_cols, ws.sorted_ids, topk,
                                (int32_t)n_in, ws.post_pad, stream);
    } else {
        rc = fg_per_token_group_quant_fp8_gather(hidden, hidden_dtype, ws.a1, ws.a1s, ws.rows, H, 128, H, H,
                                                 ws.sorted_ids, topk, (int32_t)n_in, ws.post_pad, stream);
    }
    if (rc != FG_OK) return rc;
    return run_gemms(y, ws, n_in, w1, w2, s1, s2, num_experts, H, I, topk_w, topk_w_dtype, 1, hidden_dtype, nullptr, 0,
                     nullptr, 0, 0, stream);
}

int fg_moe_routed_block_fp8_packed(void* y, const void* rows, int64_t R, int64_t row_bytes, const void* w1,
                                   const void* w2, const float* s1, const float* s2, int num_experts, int64_t H,
                                   int64_t I, void* workspace, int64_t workspace_bytes, int out_dtype,
                                   void* const* peer_out, int n_peers, int64_t peer_rows, const int32_t* n_rows_dev,
                                   int64_t region_rows, const int32_t* region_counts, int64_t region_stride,
                                   void* stream) {
    int rc = check_dims(R, num_experts, H, I, out_dtype);
    if (rc != FG_OK) return rc;
    if (R == 0) return FG_OK;
    FG_REQUIRE((y || n_peers > 0) && rows && w1 && w2 && s1 && s2 && workspace, FG_ERR_INVALID_ARGUMENT,
               "null pointer");
    FG_REQUIRE(row_bytes >= H + 4 * (H / 128) + 16 && row_bytes % 16 == 0 && (uintptr_t)rows % 16 == 0,
               FG_ERR_INVALID_ARGUMENT, "bad packed row size %lld", (long long)row_bytes);
    FG_REQUIRE((uintptr_t)workspace % 256 == 0, FG_ERR_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    const Workspace ws = carve(workspace, R, num_experts, H, I, 2);
    FG_REQUIRE(workspace_bytes >= ws.bytes, FG_ERR_INVALID_ARGUMENT, "workspace holds %lld bytes, needs %lld",
               (long long)workspace_bytes, (long long)ws.bytes);
    const uint8_t* base = reinterpret_cast<const uint8_t*>(rows);
    const int64_t s_cols = H / 128;
    const int32_t* ids = reinterpret_cast<const int32_t*>(base + H + 4 * s_cols);
    const float* wts = reinterpret_cast<const float*>(base + H + 4 * s_cols + 4);
    rc = fg_moe_align_block_size_regions(ids, 0, R, num_experts, TILE_ROWS, nullptr, 0, ws.sorted_ids, ws.max_pad,
                                         ws.expert_ids, ws.n_blocks, ws.post_pad, row_bytes / 4, 1, nullptr,
                                         n_rows_dev, region_rows, region_counts, region_stride, stream);
    if (rc != FG_OK) return rc;
    rc = fg_gather_rows_fp8(base, reinterpret_cast<const float*>(base + H), ws.a1, ws.a1s, ws.rows, H, s_cols,
                            row_bytes, row_bytes / 4, ws.sorted_ids, 1, (int32_t)R, ws.post_pad, stream);
    if (rc != FG_OK) return rc;
    const int32_t* dest = reinterpret_cast<const int32_t*>(base + H + 4 * s_cols + 8);
    return run_gemms(y, ws, R, w1, w2, s1, s2, num_experts, H, I, wts, FG_DTYPE_F32, row_bytes / 4, out_dtype,
                     n_peers > 0 ? dest : nullptr, row_bytes / 4, peer_out, n_peers, peer_rows, stream);
}

int fg_moe_routed_block_fp8_local_noalloc(void* y, const void* hidden, int hidden_dtype, const void* topk_ids,
                                          int ids_are_i64, const void* topk_w, int topk_w_dtype, int64_t T,
                                          int topk, const void* w1, const void* w2, const float* s1,
                                          const float* s2, int num_experts, int64_t H, int64_t I, void* stream) {
    int rc = check_dims(T * topk, num_experts, H, I, hidden_dtype);
    if (rc != FG_OK) return rc;
    const int64_t need = carve(nullptr, T * topk, num_experts, H, I, 2).bytes;
    FG_REQUIRE(need <= (int64_t)FG_NOALLOC_SCRATCH_BYTES, FG_ERR_UNSUPPORTED,
               "this problem (T*topk = %lld rows, %d experts, hidden %lld, intermediate %lld) needs %lld bytes of "
               "scratch; the built-in scratch holds %lld. Use fg_moe_routed_block_fp8_local with your own workspace.",
               (long long)(T * topk), num_experts, (long long)H, (long long)I, (long long)need,
               (long long)FG_NOALLOC_SCRATCH_BYTES);
    void* scratch = nullptr;
    rc = builtin_scratch(&scratch);
    if (rc != FG_OK) return rc;
    return fg_moe_routed_block_fp8_local(y, hidden, hidden_dtype, topk_ids, ids_are_i64, topk_w, topk_w_dtype, T, topk,
                                         w1, w2, s1, s2, num_experts, H, I, scratch, FG_NOALLOC_SCRATCH_BYTES, stream);
}

}  // extern "C"
