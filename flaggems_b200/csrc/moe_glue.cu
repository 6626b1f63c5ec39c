// Fused-MoE glue kernels: moe_align_block_size (one launch, thread-block cluster with
// distributed shared memory), silu_and_mul, moe_sum.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace {

// ---------------------------------------------------------------------------------------
// moe_align_block_size
//
// A cluster of up to 8 CTAs x 32 warps splits the numel route slots into contiguous
// segments, one per warp, in index order.  Each warp histograms its segment into its own
// shared-memory row; an exclusive scan over (cluster rank, warp) per expert, done through
// distributed shared memory, gives every warp the rank its first slot of each expert has
// inside that expert.  A warp then walks its segment in order, 32 slots at a time, ranking
// equal experts inside the step with match_any, so the output order inside an expert is
// ascending slot index: the same as a stable sort.  No global scratch, no global atomics.
// ---------------------------------------------------------------------------------------
constexpr int ALIGN_THREADS = 1024;
constexpr int ALIGN_WARPS = ALIGN_THREADS / 32;

struct AlignArgs {
    const void* topk_ids;
    int64_t numel;
    int num_experts;
    int block_size;
    const int32_t* expert_map;
    int expert_map_len;
    int32_t* sorted_ids;
    int64_t max_pad;
    int32_t* expert_ids;
    int64_t n_blocks;
    int32_t* num_post_pad;
    int64_t ids_stride;       // elements between consecutive ids (1 = dense)
    int32_t id_div;           // bucket = id / id_div
    int32_t* expert_counts;   // nullable: rows per bucket before padding
    const int32_t* numel_dev; // nullable: device-side slot count (numel is then the capacity)
    // Region mode (region_rows > 0): the numel slots are numel / region_rows regions of region_rows
    // slots each, and only the first region_counts[s * region_stride] slots of region s hold rows
    // (the receive buffer of the expert-parallel layer: one region per source rank).
    int64_t region_rows;
    const int32_t* region_counts;
    int64_t region_stride;
};

// Whether slot i holds a row (always, outside region mode).
__device__ __forceinline__ bool slot_present(const AlignArgs& a, int64_t i) {
    if (a.region_rows <= 0) return true;
    const int64_t s = i / a.region_rows;
    int64_t c = a.region_counts[s * a.region_stride];
    c = c < 0 ? 0 : (c > a.region_rows ? a.region_rows : c);
    return i - s * a.region_rows < c;
}

template <typename IdT>
__global__ void __launch_bounds__(ALIGN_THREADS, 1) moe_align_kernel(AlignArgs a) {
    cg::cluster_group cluster = cg::this_cluster();
    const int n_ranks = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int E = a.num_experts;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    extern __shared__ int32_t smem[];
    int32_t* warp_hist = smem;                    // [ALIGN_WARPS][E] counts, then in-CTA exclusive prefixes
    int32_t* cta_total = smem + ALIGN_WARPS * E;  // [E] this CTA's count per expert (read by peers)
    int32_t* base = cta_total + E;                // [E] first output slot for this CTA's first row of e
    int32_t* pad_lo = base + E;                   // [E] first padding slot of e
    int32_t* pad_hi = pad_lo + E;                 // [E] one past the last slot of e
    int32_t* blk_lo = pad_hi + E;                 // [E] first slot of e
    __shared__ int32_t scan_tmp[ALIGN_WARPS];
    __shared__ int32_t total_padded_s;

    for (int i = threadIdx.x; i < ALIGN_WARPS * E; i += ALIGN_THREADS) warp_hist[i] = 0;
    __syncthreads();

    // Segment of this warp: contiguous, multiple of 32 slots, in global index order.
    // Slots actually present: the host bound, or fewer when a device-side count is given (the
    // padding value stays the host bound, so "index < bound" still tells real rows from padding).
    int64_t numel = a.numel;
    if (a.numel_dev) {
        const int64_t v = *a.numel_dev;
        numel = v < 0 ? 0 : (v < numel ? v : numel);
    }
    const int64_t n_segments = (int64_t)n_ranks * ALIGN_WARPS;
    int64_t seg_len = (numel + n_segments - 1) / n_segments;
    seg_len = (seg_len + 31) / 32 * 32;
    const int64_t seg_id = (int64_t)rank * ALIGN_WARPS + warp;
    const int64_t seg_begin = seg_id * seg_len < numel ? seg_id * seg_len : numel;
    const int64_t seg_end = seg_begin + seg_len < numel ? seg_begin + seg_len : numel;
    const IdT* ids = reinterpret_cast<const IdT*>(a.topk_ids);
    int32_t* my_hist = warp_hist + warp * E;

    // Phase 1: per-warp histogram.
    for (int64_t i0 = seg_begin; i0 < seg_end; i0 += 32) {
        const int64_t i = i0 + lane;
        int e = -1;
        if (i < seg_end && slot_present(a, i)) {
            const long long v = (long long)ids[i * a.ids_stride] / a.id_div;
            if (v >= 0 && v < E) e = (int)v;
        }
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && lane == (__ffs(peers) - 1)) my_hist[e] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();

    // Phase 2a: exclusive scan over the warps of this CTA, per expert.
    for (int e = threadIdx.x; e < E; e += ALIGN_THREADS) {
        int32_t run = 0;
        for (int w = 0; w < ALIGN_WARPS; ++w) {
            const int32_t t = warp_hist[w * E + e];
            warp_hist[w * E + e] = run;
            run += t;
        }
        cta_total[e] = run;
    }
    cluster.sync();

    // Phase 2b: counts of the other CTAs through distributed shared memory.
    // Each thread owns experts e = threadIdx.x + j*ALIGN_THREADS (E <= 1024 keeps j == 0).
    int32_t before = 0, total = 0;
    const int e0 = threadIdx.x;
    if (e0 < E) {
        for (int r = 0; r < n_ranks; ++r) {
            const int32_t* peer = cluster.map_shared_rank(cta_total, r);
            const int32_t c = peer[e0];
            if (r < rank) before += c;
            total += c;
        }
    }
    cluster.sync();  // nobody may exit (or reuse cta_total) while peers still read it

    // Phase 2c: exclusive scan of the padded counts over experts (every CTA does the same).
    const int32_t bs = a.block_size;
    const int32_t padded = e0 < E ? (total + bs - 1) / bs * bs : 0;
    int32_t incl = padded;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int32_t t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) scan_tmp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int32_t v = scan_tmp[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int32_t t = __shfl_up_sync(0xffffffffu, v, o);
            if (lane >= o) v += t;
        }
        scan_tmp[lane] = v;
        if (lane == 31) total_padded_s = v;
    }
    __syncthreads();
    const int32_t offset = incl - padded + (warp > 0 ? scan_tmp[warp - 1] : 0);
    if (e0 < E) {
        base[e0] = offset + before;
        pad_lo[e0] = offset + total;
        pad_hi[e0] = offset + padded;
        blk_lo[e0] = offset;
        if (a.expert_counts && rank == 0) a.expert_counts[e0] = total;
    }
    __syncthreads();
    const int32_t total_padded = total_padded_s;

    // Phase 2d: expert id of every block, padding slots, tail.  Work is spread over the ranks; one warp
    // per expert, so that few experts with many blocks each (the expert-parallel routing pass: one
    // bucket per rank, block size 1) do not serialise on one thread.  expert_ids may be absent.
    const int32_t numel32 = (int32_t)a.numel;
    for (int e = warp + rank * ALIGN_WARPS; e < E; e += ALIGN_WARPS * n_ranks) {
        for (int32_t p = pad_lo[e] + lane; p < pad_hi[e]; p += 32) a.sorted_ids[p] = numel32;
        if (a.expert_ids) {
            int32_t id = e;
            if (a.expert_map) id = a.expert_map[e < a.expert_map_len ? e : a.expert_map_len - 1];
            for (int32_t b = blk_lo[e] / bs + lane; b < pad_hi[e] / bs; b += 32) a.expert_ids[b] = id;
        }
    }
    {
        const int64_t gtid = (int64_t)rank * ALIGN_THREADS + threadIdx.x;
        const int64_t gthreads = (int64_t)n_ranks * ALIGN_THREADS;
        for (int64_t p = total_padded + gtid; p < a.max_pad; p += gthreads) a.sorted_ids[p] = numel32;
        // Unused trailing blocks are -1; through an expert_map they become expert_map[-1],
        // i.e. its last entry, as Python indexing of the reference does.
        int32_t tail_id = -1;
        if (a.expert_map && a.expert_map_len > 0) tail_id = a.expert_map[a.expert_map_len - 1];
        if (a.expert_ids)
            for (int64_t b = total_padded / bs + gtid; b < a.n_blocks; b += gthreads) a.expert_ids[b] = tail_id;
        if (gtid == 0) a.num_post_pad[0] = total_padded;
    }

    // Phase 3: ordered scatter.  warp_hist[warp][e] is the running rank inside this CTA.
    for (int64_t i0 = seg_begin; i0 < seg_end; i0 += 32) {
        const int64_t i = i0 + lane;
        int e = -1;
        if (i < seg_end && slot_present(a, i)) {
            const long long v = (long long)ids[i * a.ids_stride] / a.id_div;
            if (v >= 0 && v < E) e = (int)v;
        }
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        const int leader = __ffs(peers) - 1;
        int32_t cur = 0;
        if (e >= 0 && lane == leader) {
            cur = my_hist[e];
            my_hist[e] = cur + __popc(peers);
        }
        cur = __shfl_sync(0xffffffffu, cur, leader);
        if (e >= 0) {
            const int32_t pos = base[e] + cur + __popc(peers & ((1u << lane) - 1u));
            a.sorted_ids[pos] = (int32_t)i;
        }
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const T* __restrict__ x, const T* __restrict__ y,
                                                           T* __restrict__ out, int64_t M, int64_t N, int64_t ld_x,
                                                           int64_t ld_y, int64_t ld_o) {
    const int64_t vec_per_row = N / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = v / vec_per_row, c = (v % vec_per_row) * 8;
        float a[8], b[8], o[8];
        fg_load8(x + r * ld_x + c, a);
        fg_load8(y + r * ld_y + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __fdividef(a[i], 1.0f + __expf(-a[i])) * b[i];
        fg_store8(out + r * ld_o + c, o);
    }
}

// Sum over the top-k slots of every token in slot order, in fp32 (the order and precision of the
// reference's moe_sum_kernel), plus an optional addend row, rounded once.  TOPK > 0: all the
// slots' 16-byte loads are issued before the first add (HBM-bound: 1 GB per step of the
// DeepSeek-V3 layer); TOPK == 0: any top-k, one load at a time.
template <typename T, int TOPK>
__global__ void __launch_bounds__(256) moe_sum_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t M,
                                                      int topk, int64_t K, const int32_t* __restrict__ row_index,
                                                      const T* __restrict__ addend) {
    const int64_t vec_per_row = K / 8;
    const int64_t total = M * vec_per_row;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = v / vec_per_row, c = (v % vec_per_row) * 8;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if constexpr (TOPK > 0) {
            uint4 raw[TOPK];
            bool have[TOPK];
#pragma unroll
            for (int k = 0; k < TOPK; ++k) {
                const int64_t src = row_index ? (int64_t)row_index[r * TOPK + k] : r * TOPK + k;
                have[k] = src >= 0;
                if constexpr (sizeof(T) == 2) {
                    raw[k] = have[k] ? __ldcs(reinterpret_cast<const uint4*>(in + src * K + c)) : make_uint4(0u, 0u, 0u, 0u);
                }
            }
            uint4 add_raw = make_uint4(0u, 0u, 0u, 0u);
            if constexpr (sizeof(T) == 2) {
                if (addend) add_raw = *reinterpret_cast<const uint4*>(addend + r * K + c);
            }
#pragma unroll
            for (int k = 0; k < TOPK; ++k) {
                if (!have[k]) continue;
                float t[8];
                if constexpr (sizeof(T) == 2) fg_unpack8<T>(raw[k], t);
                else fg_load8(in + (row_index ? (int64_t)row_index[r * TOPK + k] : r * TOPK + k) * K + c, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
            if (addend) {
                float t[8];
                if constexpr (sizeof(T) == 2) fg_unpack8<T>(add_raw, t);
                else fg_load8(addend + r * K + c, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
        } else {
            for (int k = 0; k < topk; ++k) {
                float t[8];
                const int64_t src = row_index ? (int64_t)row_index[r * topk + k] : r * topk + k;
                if (src < 0) continue;
                fg_load8(in + src * K + c, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
            if (addend) {
                float t[8];
                fg_load8(addend + r * K + c, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += t[i];
            }
        }
        fg_store8(out + r * K + c, acc);
    }
}

// Copies rows of FP8 bytes and their fp32 scale rows through an index (pure data movement).
// One warp per destination row, eight 16-byte loads per lane in flight before the first store
// (measured 142 us against 148 with four, and 158 with plain instead of streaming stores, for the
// 82688 rows of the DeepSeek-V3-shaped step: the destination is a 611 MB write stream).
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint8_t* __restrict__ src_q,
                                                          const float* __restrict__ src_s, uint8_t* __restrict__ dst_q,
                                                          float* __restrict__ dst_s, int64_t rows, int64_t K,
                                                          int64_t s_cols, int64_t src_q_stride, int64_t src_s_stride,
                                                          const int32_t* __restrict__ row_index,
                                                          int32_t index_div, int32_t index_limit,
                                                          const int32_t* __restrict__ n_rows_dev) {
    if (n_rows_dev) {
        const int64_t v = *n_rows_dev;
        rows = v < rows ? v : rows;
    }
    const int warps_per_block = blockDim.x / 32;
    const int lane = threadIdx.x & 31;
    const int nvec = (int)(K / 16);
    for (int64_t r = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5); r < rows;
         r += (int64_t)gridDim.x * warps_per_block) {
        const int32_t idx = row_index[r];
        const bool real = idx >= 0 && idx < index_limit;
        const int64_t src = real ? idx / index_div : 0;
        const uint4* sq = reinterpret_cast<const uint4*>(src_q + src * src_q_stride);
        uint4* dq = reinterpret_cast<uint4*>(dst_q + r * K);
        const float sv = (real && lane < s_cols) ? src_s[src * src_s_stride + lane] : 1.0f;
        for (int v0 = lane; v0 < nvec; v0 += 256) {
            uint4 t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int v = v0 + 32 * u;
                t[u] = (real && v < nvec) ? __ldg(sq + v) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int v = v0 + 32 * u;
                if (v < nvec) __stcs(dq + v, t[u]);
            }
        }
        if (lane < s_cols) dst_s[r * s_cols + lane] = sv;
        for (int64_t v = lane + 32; v < s_cols; v += 32) dst_s[r * s_cols + v] = real ? src_s[src * src_s_stride + v] : 1.0f;
    }
}

// Group of every row from the ends of the groups: ids[r] = number of offsets <= r (rows past the last
// end get num_groups, which the alignment kernel ignores).
__global__ void __launch_bounds__(256) group_ids_kernel(const int32_t* __restrict__ offs, int num_groups, int64_t rows,
                                                        int32_t* __restrict__ ids) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
        int lo = 0, hi = num_groups;  // first g with offs[g] > r
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if ((int64_t)offs[mid] > r) hi = mid;
            else lo = mid + 1;
        }
        ids[r] = lo;
    }
}

unsigned grid_for(int64_t work_items, int per_block) {
    int64_t b = fg_cdiv(work_items, per_block);
    const int64_t cap = (int64_t)fg_num_sms() * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (unsigned)b;
}

}  // namespace

extern "C" {

int fg_moe_align_block_size(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts, int block_size,
                            const int32_t* expert_map, int expert_map_len, int32_t* sorted_ids, int64_t max_pad,
                            int32_t* expert_ids, int64_t n_blocks, int32_t* num_post_pad, void* stream) {
    return fg_moe_align_block_size_ex(topk_ids, ids_are_i64, numel, num_experts, block_size, expert_map,
                                      expert_map_len, sorted_ids, max_pad, expert_ids, n_blocks, num_post_pad, 1, 1,
                                      nullptr, nullptr, stream);
}

int fg_moe_align_block_size_ex(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts, int block_size,
                               const int32_t* expert_map, int expert_map_len, int32_t* sorted_ids, int64_t max_pad,
                               int32_t* expert_ids, int64_t n_blocks, int32_t* num_post_pad, int64_t ids_stride,
                               int id_div, int32_t* expert_counts, const int32_t* numel_dev, void* stream) {
    return fg_moe_align_block_size_regions(topk_ids, ids_are_i64, numel, num_experts, block_size, expert_map,
                                           expert_map_len, sorted_ids, max_pad, expert_ids, n_blocks, num_post_pad,
                                           ids_stride, id_div, expert_counts, numel_dev, 0, nullptr, 0, stream);
}

int fg_moe_align_block_size_regions(const void* topk_ids, int ids_are_i64, int64_t numel, int num_experts,
                                    int block_size, const int32_t* expert_map, int expert_map_len, int32_t* sorted_ids,
                                    int64_t max_pad, int32_t* expert_ids, int64_t n_blocks, int32_t* num_post_pad,
                                    int64_t ids_stride, int id_div, int32_t* expert_counts, const int32_t* numel_dev,
                                    int64_t region_rows, const int32_t* region_counts, int64_t region_stride,
                                    void* stream) {
    FG_REQUIRE(region_rows >= 0 && (region_rows == 0 || (region_counts && region_stride >= 1 && numel % region_rows == 0)),
               FG_ERR_INVALID_ARGUMENT, "region mode needs counts, a stride >= 1 and numel divisible by region_rows");
    FG_REQUIRE(ids_stride >= 1 && id_div >= 1, FG_ERR_INVALID_ARGUMENT, "ids_stride and id_div must be >= 1");
    FG_REQUIRE(numel >= 0 && num_experts > 0 && block_size > 0, FG_ERR_INVALID_ARGUMENT,
               "numel %lld, num_experts %d, block_size %d", (long long)numel, num_experts, block_size);
    FG_REQUIRE(num_experts <= ALIGN_THREADS, FG_ERR_UNSUPPORTED, "num_experts %d exceeds the supported maximum %d",
               num_experts, ALIGN_THREADS);
    FG_REQUIRE(numel + (int64_t)num_experts * block_size < (1ll << 31), FG_ERR_UNSUPPORTED, "numel too large");
    // At most min(numel, E) experts are non-empty and only those are padded.
    int64_t need_pad = numel + (int64_t)num_experts * (block_size - 1);
    if (numel * block_size < need_pad) need_pad = numel * block_size;
    FG_REQUIRE(max_pad >= need_pad, FG_ERR_INVALID_ARGUMENT,
               "sorted_ids holds %lld entries, needs at least min(numel*block_size, numel + E*(block_size-1)) = %lld",
               (long long)max_pad, (long long)need_pad);
    FG_REQUIRE(expert_ids == nullptr || n_blocks >= need_pad / block_size, FG_ERR_INVALID_ARGUMENT,
               "expert_ids holds %lld entries, needs %lld", (long long)n_blocks, (long long)(need_pad / block_size));
    FG_REQUIRE(sorted_ids && num_post_pad && (topk_ids || numel == 0), FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE(expert_map == nullptr || expert_map_len >= num_experts, FG_ERR_INVALID_ARGUMENT,
               "expert_map has %d entries for %d experts", expert_map_len, num_experts);

    AlignArgs a{topk_ids, numel, num_experts, block_size, expert_map, expert_map_len,
                sorted_ids, max_pad, expert_ids, n_blocks, num_post_pad, ids_stride, id_div, expert_counts, numel_dev,
                region_rows, region_counts, region_stride};
    // One CTA handles 32 warps x 128 slots comfortably; grow the cluster with numel up to 8.
    int ranks = 1;
    while (ranks < 8 && (int64_t)ranks * ALIGN_THREADS * 4 < numel) ranks *= 2;
    const size_t smem = (size_t)(ALIGN_WARPS + 5) * num_experts * sizeof(int32_t);

    auto kernel = ids_are_i64 ? moe_align_kernel<int64_t> : moe_align_kernel<int32_t>;
    // Opt in to large dynamic shared memory once per device, kernel and size (a per-device
    // attribute, kept out of the steady-state call path).
    static std::mutex mu;
    static size_t smem_set[64][2];
    {
        const int dev = fg_device_index();
        std::lock_guard<std::mutex> lock(mu);
        size_t& have = smem_set[dev][ids_are_i64 ? 1 : 0];
        if (have < 48 * 1024) have = 48 * 1024;
        if (smem > have) {
            FG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            have = smem;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ranks, 1, 1);
    cfg.blockDim = dim3(ALIGN_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ranks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FG_CUDA(cudaLaunchKernelEx(&cfg, kernel, a));
    fg_count_launch(1);
    return FG_OK;
}

int fg_group_ids_from_offsets(const int32_t* offs, int num_groups, int64_t rows, int32_t* ids, void* stream) {
    FG_REQUIRE(num_groups > 0 && rows >= 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    if (rows == 0) return FG_OK;
    FG_REQUIRE(offs && ids, FG_ERR_INVALID_ARGUMENT, "null pointer");
    group_ids_kernel<<<grid_for(rows, 256), 256, 0, (cudaStream_t)stream>>>(offs, num_groups, rows, ids);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_silu_and_mul(const void* x, const void* y, void* out, int64_t M, int64_t N, int64_t ld_x, int64_t ld_y,
                    int64_t ld_out, int dtype, void* stream) {
    FG_REQUIRE(M >= 0 && N >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    if (M == 0 || N == 0) return FG_OK;
    const int esz = dtype == FG_DTYPE_F32 ? 4 : 2;
    FG_REQUIRE(N % 8 == 0 && (ld_x * esz) % 16 == 0 && (ld_y * esz) % 16 == 0 && (ld_out * esz) % 16 == 0 &&
                   (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)out % 16 == 0,
               FG_ERR_UNSUPPORTED, "silu_and_mul needs N %% 8 == 0 and 16-byte aligned rows");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = grid_for(M * (N / 8), 256);
    switch (dtype) {
        case FG_DTYPE_BF16:
            silu_and_mul_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)y,
                                                      (__nv_bfloat16*)out, M, N, ld_x, ld_y, ld_out);
            break;
        case FG_DTYPE_F16:
            silu_and_mul_kernel<<<grid, 256, 0, st>>>((const __half*)x, (const __half*)y, (__half*)out, M, N, ld_x,
                                                      ld_y, ld_out);
            break;
        case FG_DTYPE_F32:
            silu_and_mul_kernel<<<grid, 256, 0, st>>>((const float*)x, (const float*)y, (float*)out, M, N, ld_x, ld_y,
                                                      ld_out);
            break;
        default: fg_set_error("unsupported dtype code %d", dtype); return FG_ERR_INVALID_ARGUMENT;
    }
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_moe_sum_indexed(const void* in, void* out, int64_t M, int topk, int64_t K, int dtype,
                       const int32_t* row_index, const void* addend, void* stream) {
    FG_REQUIRE(M >= 0 && K >= 0 && topk >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    if (M == 0 || K == 0) return FG_OK;
    FG_REQUIRE(K % 8 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)addend % 16 == 0,
               FG_ERR_UNSUPPORTED, "moe_sum needs K %% 8 == 0 and 16-byte aligned buffers");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = grid_for(M * (K / 8), 256);
    auto launch = [&](auto tag) {
        using T = decltype(tag);
        const T* i = (const T*)in;
        T* o = (T*)out;
        const T* a = (const T*)addend;
        switch (topk) {
            case 2: moe_sum_kernel<T, 2><<<grid, 256, 0, st>>>(i, o, M, topk, K, row_index, a); break;
            case 4: moe_sum_kernel<T, 4><<<grid, 256, 0, st>>>(i, o, M, topk, K, row_index, a); break;
            case 6: moe_sum_kernel<T, 6><<<grid, 256, 0, st>>>(i, o, M, topk, K, row_index, a); break;
            case 8: moe_sum_kernel<T, 8><<<grid, 256, 0, st>>>(i, o, M, topk, K, row_index, a); break;
            default: moe_sum_kernel<T, 0><<<grid, 256, 0, st>>>(i, o, M, topk, K, row_index, a); break;
        }
    };
    switch (dtype) {
        case FG_DTYPE_BF16: launch(__nv_bfloat16()); break;
        case FG_DTYPE_F16: launch(__half()); break;
        case FG_DTYPE_F32: launch(float()); break;
        default: fg_set_error("unsupported dtype code %d", dtype); return FG_ERR_INVALID_ARGUMENT;
    }
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_moe_sum(const void* in, void* out, int64_t M, int topk, int64_t K, int dtype, void* stream) {
    return fg_moe_sum_indexed(in, out, M, topk, K, dtype, nullptr, nullptr, stream);
}

int fg_gather_rows_fp8(const void* src_q, const float* src_s, void* dst_q, float* dst_s, int64_t rows, int64_t K,
                       int64_t s_cols, int64_t src_q_stride, int64_t src_s_stride, const int32_t* row_index,
                       int32_t index_div, int32_t index_limit, const int32_t* n_rows_dev, void* stream) {
    FG_REQUIRE(src_q_stride >= K && src_q_stride % 16 == 0 && src_s_stride >= s_cols, FG_ERR_INVALID_ARGUMENT,
               "bad source strides");
    FG_REQUIRE(rows >= 0 && K >= 0 && s_cols >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    if (rows == 0) return FG_OK;
    FG_REQUIRE(src_q && dst_q && row_index && index_div > 0 && (s_cols == 0 || (src_s && dst_s)),
               FG_ERR_INVALID_ARGUMENT, "null pointer or bad index_div");
    FG_REQUIRE(K % 16 == 0 && (uintptr_t)src_q % 16 == 0 && (uintptr_t)dst_q % 16 == 0, FG_ERR_UNSUPPORTED,
               "gather_rows needs K %% 16 == 0 and 16-byte aligned buffers");
    int64_t blocks = fg_cdiv(rows, 8);
    const int64_t cap = (int64_t)fg_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    gather_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
        (const uint8_t*)src_q, src_s, (uint8_t*)dst_q, dst_s, rows, K, s_cols, src_q_stride, src_s_stride, row_index,
        index_div, index_limit, n_rows_dev);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

}  // extern "C"
