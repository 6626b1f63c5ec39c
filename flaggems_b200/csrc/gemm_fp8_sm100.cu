// FP8 (e4m3) scaled matrix products on tcgen05 tensor cores for sm_100a.
//
// One persistent, warp-specialised kernel template serves the dense scaled GEMM
// (scalar / per-row / per-column scales), the 128x128 block-scaled GEMM and the grouped
// expert GEMMs of the fused MoE layer:
//
//   warp 0      TMA producer: A tile [128 x 128 B] and B tile [BN x 128 B] per K block into a
//               multi-stage shared-memory ring (128-byte swizzle), mbarrier complete_tx.
//   warp 1      MMA issuer: tcgen05.mma kind::f8f6f4, M=128, N=BN, K=32 per instruction, fp32
//               accumulators in TMEM (two buffers of BN columns), tcgen05.commit to release
//               ring stages and to publish accumulators.  The warp stays converged and an
//               elected lane issues; barrier states are probed one K block ahead.
//   warps 4..   epilogue: tcgen05.ld TMEM -> registers, scales / SiLU / router weight / bias,
//               conversion and global stores.  BN/32 warps (one or two warpgroups); each thread
//               owns one tile row and 128 accumulator columns.  (Warps 2-3 only pad the first
//               warpgroup so that setmaxnreg can move registers from it to the epilogue.)
//
// Block-scaled mode: the accumulator of every 128-wide K block is published separately and
// the epilogue warps fold it into fp32 registers as acc += partial * (As[m,kb] * Bs[nb,kb])
// while the MMA warp fills the other TMEM buffer.
//
// Large dense products use the CTA-pair form of the same kernel (cta_group::2, one 256 x 256
// tile per two SMs); decode-sized M uses the split-K form (one cluster per tile).
//
// Every mbarrier wait is bounded; a wait that runs out sets the device status word and the
// CTA drains and frees its TMEM instead of hanging.
#include <cooperative_groups.h>
#include <cuda.h>
#include <stdlib.h>
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "ptx_sm100.cuh"

using namespace fgptx;
namespace cg = cooperative_groups;

// Optional stall accounting for kernel development (-DFG_GEMM_PROFILE; never in the shipped build):
// per CTA, cycles the producer, the MMA warp and one epilogue warp spend in each of their waits.
#ifdef FG_GEMM_PROFILE
__device__ long long g_gemm_prof[256 * 12];
#define FG_PROF_DECL(name) long long name = 0
#define FG_PROF_T0(t) const long long t = clock64()
#define FG_PROF_ADD(acc, t) acc += clock64() - t
#define FG_PROF_OUT(slot, v) if (blockIdx.x < 256) g_gemm_prof[blockIdx.x * 12 + (slot)] = (v)
#else
#define FG_PROF_DECL(name)
#define FG_PROF_T0(t)
#define FG_PROF_ADD(acc, t)
#define FG_PROF_OUT(slot, v)
#endif

namespace {

constexpr int BLOCK_M = 128;
constexpr int BLOCK_K = 128;  // e4m3: bytes == elements; one 128-byte swizzle row
constexpr int UMMA_K = 32;
constexpr int GROUP_M = 16;  // m-blocks per rasterisation band

struct GemmParams {
    int64_t M;  // dense: rows of A and C.  grouped: rows available in A (upper bound)
    int N;      // rows of B per expert (fused SiLU: 2*I)
    int K;
    int n_out;  // columns written (N, or I with fused SiLU)
    void* c;
    int64_t ld_c;
    int out_dtype;
    int bias_dtype;  // element type of bias (the output type, or fp32 when the output is e4m3 / for grouped mm)
    int64_t bias_stride_e;  // grouped: elements between the bias rows of consecutive experts (0: one row)
    int c_vec_ok;  // rows of C are 16-byte aligned
    const float* sa;
    const float* sb;
    const void* bias;
    int sa_mode, sb_mode;  // FG_SCALE_SCALAR / FG_SCALE_VECTOR (ignored in block mode)
    int bias_after_round;
    int64_t ld_as, as_stride_k;                     // block mode: row / K-block strides of As
    int64_t bs_stride_n, bs_stride_k, bs_stride_e;  // block mode: strides of Bs
    int64_t sb_stride_e;                            // vector mode: per-expert stride of sb
    int grouped;
    int int8;  // operand kind: 0 e4m3, 1 signed 8-bit integers (accumulators int32), 2 bf16, 3 f16 (K then counts bytes)
    const int32_t* sorted_ids;
    const int32_t* expert_ids;
    const int32_t* num_post_pad;
    int block_rows;  // grouped: rows per m-tile (TMA box rows of A), <= 128
    int a_box_rows;  // dense: TMA box rows of A (128, or fewer when M is small)
    int64_t numel;
    int scatter, mul_weight;
    const void* topk_w;
    int topk_w_dtype;
    int64_t topk_w_stride;  // elements between the weights of consecutive route slots
    // Peer scatter (expert-parallel combine fused into GEMM2's epilogue): row with arrival index
    // sid is stored to peer_out[dest[sid*dest_stride + 1]] at row dest[sid*dest_stride].
    const int32_t* dest;
    int64_t dest_stride;
    int n_peers;
    int64_t peer_rows;  // rows each peer buffer holds; a row addressed outside is dropped and reported
    void* peer_out[8];
    unsigned int* status;
};

// PAIR: two CTAs of a cluster (cta_group::2) compute one 256 x 256 tile.  Each stages its own 128
// rows of A and 128 of the 256 rows of B, and holds the accumulator of its 128 rows in its TMEM;
// one MMA instruction issued by the even CTA drives both tensor cores.  Per CTA and K block that
// is 32 KB through L2 and shared memory instead of 48 KB for the same arithmetic.
// ASTORE (block-scaled 256-wide tiles with 16-bit outputs): at the end of a tile the epilogue warps
// only convert their accumulators and park the tile in shared memory; a store warp writes it to
// global (or peer) memory while the epilogue warps are already folding the next tile's K blocks.
// In block-scaled mode those warps are needed in every K block, so whatever they do at a tile's end
// stalls the tensor core once its two accumulator buffers are full.  The parked tile takes the
// room of one ring stage (three stages instead of four).
template <int BN, bool SMALL_A, bool PAIR = false, bool ASTORE = false>
struct Cfg {
    static_assert(!ASTORE || (BN == 256 && !SMALL_A && !PAIR), "the store warp serves the 256-wide tile");
    static_assert(BN == 32 || BN == 64 || BN == 128 || BN == 256, "unsupported tile width");
    static_assert(!SMALL_A || BN == 32, "the narrow-A layout exists for the 32-wide tile only");
    static_assert(!PAIR || BN == 256, "the CTA-pair layout is built for the 256-wide tile");
    static constexpr int COLS = BN >= 128 ? 128 : BN;          // accumulator columns per epilogue thread
    static constexpr int EPI_WARPS = BN >= 128 ? BN / 32 : 4;  // one warp per 32 TMEM lanes, x column halves
    static constexpr int FIRST_EPI_WARP = 4;  // warps 0-3: TMA, MMA, two spare (one warpgroup)
    static constexpr int THREADS = 32 * (FIRST_EPI_WARP + EPI_WARPS);
    // With 384 threads the launch-time register file share is 168 per thread; the epilogue
    // warpgroups raise theirs with setmaxnreg after the producer warpgroup has shrunk its own.
    // The pool is what the CTA got at launch (384 x 168 = 64512), and setmaxnreg.inc blocks
    // until the pool can pay: 128 x REGS_PRODUCER + 256 x REGS_EPILOGUE must not exceed it.
    static constexpr bool REBALANCE_REGS = BN == 256;
    static constexpr int REGS_PRODUCER = 40, REGS_EPILOGUE = 232;
    static_assert(128 * REGS_PRODUCER + 256 * REGS_EPILOGUE <= 384 * 168, "setmaxnreg.inc would wait forever");
    // Narrow-A layout (M <= 32, weight streaming): only 32 rows of A are staged per K block.  The
    // MMA still reads 128 rows from the stage's address; rows 32..127 are whatever follows in
    // shared memory (later stages or the tail pad) and only feed accumulator rows nobody reads.
    static constexpr int A_ROWS_SMEM = SMALL_A ? 32 : BLOCK_M;
    static constexpr int A_BYTES = A_ROWS_SMEM * BLOCK_K;
    static constexpr int B_BYTES = (PAIR ? BN / 2 : BN) * BLOCK_K;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = ASTORE ? 3 : PAIR ? 6 : BN == 256 ? 4 : BN == 128 ? 6 : BN == 64 ? 8 : (SMALL_A ? 22 : 9);
    static constexpr int PARK_BYTES = ASTORE ? BLOCK_M * BN * 2 + BLOCK_M * 8 : 0;  // parked tile + one pointer per row
    static constexpr int TAIL_PAD = SMALL_A ? BLOCK_M * BLOCK_K : 0;
    static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int BAR_BYTES = 512;  // (2*STAGES + 6) mbarriers, TMEM base slot, abort flag, turn counter
    static_assert((2 * STAGES + 6) * 8 + 16 <= BAR_BYTES, "barrier area too small");
    static constexpr int EPI_STAGE_BYTES = 2048;  // per epilogue warp: 32 rows x 64 bytes
    static constexpr int SMEM_BYTES =
        STAGES * STAGE_BYTES + TAIL_PAD + BAR_BYTES + EPI_WARPS * EPI_STAGE_BYTES + PARK_BYTES + 1024;
    static_assert(SMEM_BYTES <= 232448, "over the 227 KB shared memory limit");
    // split-K parks a 128 x BN fp32 partial tile (rows padded by 4 floats) in the ring's memory
    static_assert(SMALL_A || PAIR || BLOCK_M * (BN + 4) * 4 <= STAGES * STAGE_BYTES, "partial tile does not fit");
};

__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
    if (dtype == FG_DTYPE_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
    if (dtype == FG_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
    return reinterpret_cast<const float*>(p)[i];
}

__device__ __forceinline__ float round_through(float v, int dtype) {
    if (dtype == FG_DTYPE_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    if (dtype == FG_DTYPE_F16) return __half2float(__float2half_rn(v));
    return v;
}

__host__ __device__ __forceinline__ int out_elem_size(int dtype) {
    return dtype == FG_DTYPE_F32 ? 4 : (dtype == FG_DTYPE_E4M3 ? 1 : 2);
}

__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// Stores 32 consecutive output values of one row; ncols (<= 32) of them are in range.
__device__ __forceinline__ void store_chunk(void* row_ptr, int col0, const float (&v)[32], int ncols, int dtype,
                                            bool vec_ok) {
    if (dtype == FG_DTYPE_F32) {
        float* o = reinterpret_cast<float*>(row_ptr) + col0;
        if (vec_ok && ncols == 32) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(o)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < ncols) o[i] = v[i];
        }
        return;
    }
    if (dtype == FG_DTYPE_E4M3) {
        // round to nearest even, saturating at +-448 (cvt.rn.satfinite.e4m3x2.f32)
        uint32_t b[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i], v[4 * i + 1]), __NV_SATFINITE, __NV_E4M3);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2], v[4 * i + 3]), __NV_SATFINITE, __NV_E4M3);
            b[i] = lo | (hi << 16);
        }
        uint8_t* o = reinterpret_cast<uint8_t*>(row_ptr) + col0;
        if (vec_ok && ncols == 32) {
            reinterpret_cast<uint4*>(o)[0] = make_uint4(b[0], b[1], b[2], b[3]);
            reinterpret_cast<uint4*>(o)[1] = make_uint4(b[4], b[5], b[6], b[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < ncols) o[i] = (uint8_t)((b[i >> 2] >> (8 * (i & 3))) & 0xffu);
        }
        return;
    }
    uint32_t w[16];
    if (dtype == FG_DTYPE_BF16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    uint16_t* o = reinterpret_cast<uint16_t*>(row_ptr) + col0;
    if (vec_ok && ncols == 32) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(o)[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < ncols) o[i] = (uint16_t)((i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xffffu));
    }
}

// Stores 32 consecutive 16-bit output values per lane (lane = row) with coalescing: the warp
// transposes the 32 x 64-byte block through its private shared-memory staging area (16-byte
// chunks XOR-swizzled so that neither side has bank conflicts) and then writes 64 contiguous
// bytes per row, eight rows per instruction, instead of 16 bytes to 32 different rows.  That is
// what makes the stores to a peer GPU's memory (fused combine) efficient on NVLink, and it halves
// the number of partial-sector writes for local outputs.  All 32 lanes must call it.
__device__ __forceinline__ void store_chunk_coalesced(uint8_t* stage, int lane, const float (&v)[32],
                                                      uint8_t* my_row_ptr, bool my_row_ok, int col0, int dtype) {
    uint32_t w[16];
    if (dtype == FG_DTYPE_BF16) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
    }
    const int wsw = (lane >> 1) & 3;
#pragma unroll
    for (int k = 0; k < 4; ++k)
        *reinterpret_cast<uint4*>(stage + lane * 64 + ((k ^ wsw) << 4)) =
            make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
    __syncwarp();
    const int c = lane & 3;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int r = (lane >> 2) + 8 * j;
        const uint4 val = *reinterpret_cast<const uint4*>(stage + r * 64 + ((c ^ ((r >> 1) & 3)) << 4));
        const unsigned long long ptr = __shfl_sync(0xffffffffu, (unsigned long long)my_row_ptr, r);
        const int ok = __shfl_sync(0xffffffffu, (int)my_row_ok, r);
        if (ok) *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(ptr) + (size_t)col0 * 2 + (c << 4)) = val;
    }
    __syncwarp();
}

struct TileCoord {
    int m_blk, n_blk;
};

__device__ __forceinline__ TileCoord tile_coord(int t, int num_m, int num_n) {
    const int band = t / (GROUP_M * num_n);
    const int first_m = band * GROUP_M;
    const int gm = min(GROUP_M, num_m - first_m);
    const int rem = t - band * GROUP_M * num_n;
    TileCoord tc;
    tc.m_blk = first_m + rem % gm;
    tc.n_blk = rem / gm;
    return tc;
}

// SPLITK: the CTAs of one thread-block cluster share an output tile and split its K range; each
// leaves its fp32 partial tile in its own shared memory and the cluster adds them up through
// distributed shared memory (no global scratch, no atomics).  For decode-sized M, where there are
// fewer tiles than SMs and the job is to pull the weights from HBM with every SM.
// OPK (operand kind): 0 = e4m3 (kind::f8f6f4); 1 = signed 8-bit integers with 32-bit integer accumulators
// (kind::i8) for the int8 w8a8 expert GEMMs (the epilogue converts the accumulators to fp32 and applies
// the per-row x per-column scales); 2 / 3 = bf16 / f16 (kind::f16) for the unquantised and
// weight-only-quantised expert GEMMs.  The main loop is written in bytes (a K block is 128 bytes of a
// K-major row, an MMA consumes 32 of them), so a 16-bit product of K elements runs as 2K bytes.
template <int BN, bool BLOCK_SCALED, bool FUSE_SILU, bool SMALL_A, bool SPLITK, bool PAIR = false, bool ASTORE = false,
          int OPK = 0>
__global__ void __launch_bounds__(Cfg<BN, SMALL_A, PAIR, ASTORE>::THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                const GemmParams p) {
    using C = Cfg<BN, SMALL_A, PAIR, ASTORE>;
    static_assert(!ASTORE || (BLOCK_SCALED && !SPLITK), "the store warp serves the block-scaled tiles");
    constexpr bool INT8 = OPK == 1;
    static_assert(OPK == 0 || (!BLOCK_SCALED && !SPLITK && !PAIR && !SMALL_A), "int8 and 16-bit operands serve the plain and grouped tiles");
    // accumulator word -> fp32
    auto acc_f = [](uint32_t raw) -> float {
        if constexpr (INT8) return __int2float_rn((int)raw);
        else return __uint_as_float(raw);
    };
    static_assert(!SPLITK || (!FUSE_SILU && !SMALL_A && BN >= 128), "split-K is built for the plain wide tiles");
    static_assert(!PAIR || (!SPLITK && !FUSE_SILU && !SMALL_A), "the CTA pair serves the plain dense tiles");
    static_assert(!FUSE_SILU || BN >= 128, "fused SiLU needs a tile of at least 128 columns");
    constexpr int STAGES = C::STAGES;
    constexpr int OUT_TILE_N = FUSE_SILU ? BN / 2 : BN;  // output columns per tile
    // DUAL (block-scaled wide tiles): warps 1 and 2 issue the MMAs of alternate K blocks.  A K block's
    // trip through the issuing warp (two barrier waits of ~100 cycles each even when they are already
    // complete, four MMAs at ~46 cycles of issue each, two commits) measured ~530 cycles, more than
    // the 512 cycles the tensor core needs for the block, so one warp starves it.  In block-scaled
    // mode every K block has its own accumulator buffer (block j -> buffer j & 1), so the two warps
    // never accumulate into the same buffer and need no ordering beyond a turn counter that keeps
    // the tensor core's queue in K-block order.
    constexpr bool DUAL = BLOCK_SCALED && !PAIR && !SMALL_A && !SPLITK && BN == 256;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * C::STAGE_BYTES + C::TAIL_PAD);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full = empty_bar + STAGES;
    uint64_t* tmem_empty = tmem_full + 2;
    uint64_t* park_full = tmem_empty + 2;   // ASTORE: the parked tile is complete (all epilogue warps)
    uint64_t* park_free = park_full + 1;    // ASTORE: the store warp has written it out
    uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(park_free + 1);
    volatile uint32_t* abort_flag = tmem_base_slot + 1;
    volatile uint32_t* issued_blocks = tmem_base_slot + 2;  // DUAL: K blocks whose MMAs have been issued
    uint8_t* epi_stage_base = smem + STAGES * C::STAGE_BYTES + C::TAIL_PAD + C::BAR_BYTES;
    uint8_t* park_tile = epi_stage_base + C::EPI_WARPS * C::EPI_STAGE_BYTES;        // [128][OUT_TILE_N] 16-bit, swizzled
    unsigned long long* park_rows = reinterpret_cast<unsigned long long*>(park_tile + BLOCK_M * BN * 2);  // row pointers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;  // 0: issues the MMAs, owns the shared barriers

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], PAIR ? 2 * C::EPI_WARPS : C::EPI_WARPS);
        }
        mbar_init(park_full, C::EPI_WARPS);
        mbar_init(park_free, 1);
        *abort_flag = 0u;
        *issued_blocks = 0u;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_base_slot, C::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    if constexpr (PAIR) cluster_sync_all();  // the peer's barriers exist before anything signals them
    else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_base_slot;

    const int num_k_blocks = (p.K + BLOCK_K - 1) / BLOCK_K;
    int num_m;
    if (p.grouped) {
        int64_t rows = *p.num_post_pad;
        if (rows > p.M) rows = p.M;
        num_m = (int)(rows / p.block_rows);
    } else {
        num_m = (int)((p.M + BLOCK_M - 1) / BLOCK_M);
    }
    if constexpr (PAIR) num_m = (int)((p.M + 2 * BLOCK_M - 1) / (2 * BLOCK_M));
    const int num_n = (p.n_out + OUT_TILE_N - 1) / OUT_TILE_N;
    const int num_tiles = num_m * num_n;
    const int a_rows_step = PAIR ? 2 * BLOCK_M : (p.grouped ? p.block_rows : BLOCK_M);
    // K range and tile walk of this CTA (split-K: rank in the cluster = K slice, one cluster per tile)
    int kb_begin = 0, kb_end = num_k_blocks, tile_first = blockIdx.x, tile_step = gridDim.x, k_slices = 1;
    if constexpr (PAIR) {
        tile_first = blockIdx.x / 2;
        tile_step = gridDim.x / 2;
    }
    if constexpr (SPLITK) {
        cg::cluster_group cluster = cg::this_cluster();
        k_slices = (int)cluster.num_blocks();
        const int per = (num_k_blocks + k_slices - 1) / k_slices;
        kb_begin = (int)cluster.block_rank() * per;
        kb_end = min(kb_begin + per, num_k_blocks);
        tile_first = blockIdx.x / k_slices;
        tile_step = gridDim.x / k_slices;
    }
    const uint32_t stage_tx = (uint32_t)((p.grouped ? p.block_rows : p.a_box_rows) * BLOCK_K + C::B_BYTES);

    if (warp < C::FIRST_EPI_WARP) {
      if constexpr (C::REBALANCE_REGS) setmaxnreg_dec<C::REGS_PRODUCER>();
      if (warp == 0) {
        // ------------------------------- TMA producer -------------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            FG_PROF_DECL(prof_wait);
            for (int t = tile_first; t < num_tiles && ok; t += tile_step) {
                const TileCoord tc = tile_coord(t, num_m, num_n);
                const int expert = p.grouped ? p.expert_ids[tc.m_blk] : 0;
                if (expert < 0) continue;
                const int m0 = tc.m_blk * a_rows_step + (int)cta_rank * BLOCK_M;
                const int n0 = tc.n_blk * OUT_TILE_N;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    FG_PROF_T0(tw);
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, p.status, 1);
                    FG_PROF_ADD(prof_wait, tw);
                    if (!ok) break;
                    uint8_t* sa = smem + stage * C::STAGE_BYTES;
                    uint8_t* sb = sa + C::A_BYTES;
                    if constexpr (PAIR) {
                        // Both CTAs' loads complete on the even CTA's barrier, which expects the
                        // bytes of both; a completion that gets there before the expect only drives
                        // the count negative for a moment.
                        const uint32_t bar0 = mapa_shared(smem_u32(&full_bar[stage]), 0u);
                        if (cta_rank == 0) mbar_arrive_expect_tx(&full_bar[stage], 2u * stage_tx);
                        tma_load_2d_2cta(sa, &tm_a, bar0, kb * BLOCK_K, m0);
                        tma_load_3d_2cta(sb, &tm_b, bar0, kb * BLOCK_K, n0 + (int)cta_rank * (BN / 2), 0);
                        if (++stage == STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                        continue;
                    }
                    mbar_arrive_expect_tx(&full_bar[stage], stage_tx);
                    tma_load_2d(sa, &tm_a, &full_bar[stage], kb * BLOCK_K, m0);
                    if constexpr (FUSE_SILU) {
                        tma_load_3d(sb, &tm_b, &full_bar[stage], kb * BLOCK_K, n0, expert);
                        tma_load_3d(sb + (BN / 2) * BLOCK_K, &tm_b, &full_bar[stage], kb * BLOCK_K, p.N / 2 + n0,
                                    expert);
                    } else {
                        tma_load_3d(sb, &tm_b, &full_bar[stage], kb * BLOCK_K, n0, expert);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            FG_PROF_OUT(0, prof_wait);
        }
    } else if (ASTORE && warp == 3) {
        // ------------------------------- store warp -----------------------------------------
        // Writes parked tiles out: one 16-byte piece per lane, a whole row (or two) per instruction,
        // to the row's own destination (plain, scattered or on a peer GPU).
        constexpr int ROW_BYTES = OUT_TILE_N * 2;
        constexpr int LANES_PER_ROW = ROW_BYTES / 16;      // 32 or 16
        constexpr int ROWS_PER_STEP = 32 / LANES_PER_ROW;  // 1 or 2
        uint32_t it = 0;
        bool ok = true;
        for (int t = tile_first; t < num_tiles && ok; t += tile_step) {
            const TileCoord tc = tile_coord(t, num_m, num_n);
            const int expert = p.grouped ? p.expert_ids[tc.m_blk] : 0;
            if (expert < 0) continue;
            const int n0 = tc.n_blk * OUT_TILE_N;
            ok = __all_sync(0xffffffffu, mbar_wait(park_full, it & 1u, abort_flag, p.status, 8));
            if (!ok) break;
            const int sub = lane / LANES_PER_ROW, q = lane % LANES_PER_ROW;
#pragma unroll 4
            for (int r0 = 0; r0 < BLOCK_M; r0 += ROWS_PER_STEP) {
                const int r = r0 + sub;
                const unsigned long long dst = park_rows[r];
                const int col = n0 + ((q ^ (r & 7)) << 3);
                if (dst != 0ull && col < p.n_out) {
                    const uint4 v = *reinterpret_cast<const uint4*>(park_tile + r * ROW_BYTES + (q << 4));
                    *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(dst) + (size_t)col * 2) = v;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(park_free);
            ++it;
        }
    } else if (DUAL && (warp == 1 || warp == 2)) {
        // ------------------------------- MMA issuers, alternate K blocks ----------------------
        constexpr uint32_t idesc = umma_idesc_e4m3_f32(BLOCK_M, BN);
        const uint32_t me = (uint32_t)(warp - 1);
        uint32_t j = 0;  // K blocks of this CTA so far, over all its tiles
        bool ok = true;
        FG_PROF_DECL(prof_tmem);
        FG_PROF_DECL(prof_full);
        FG_PROF_DECL(prof_turn);
        FG_PROF_DECL(prof_blocks);
        FG_PROF_T0(prof_start);
        for (int t = tile_first; t < num_tiles && ok; t += tile_step) {
            const TileCoord tc = tile_coord(t, num_m, num_n);
            const int expert = p.grouped ? p.expert_ids[tc.m_blk] : 0;
            if (expert < 0) continue;
            for (int kb = kb_begin; kb < kb_end && ok; ++kb, ++j) {
                if ((j & 1u) != me) continue;
                const uint32_t stage = j % STAGES, phase = (j / STAGES) & 1u;
                FG_PROF_T0(tw);
                ok = __all_sync(0xffffffffu, mbar_wait(&tmem_empty[me], ((j >> 1) & 1u) ^ 1u, abort_flag, p.status, 2));
                FG_PROF_ADD(prof_tmem, tw);
                if (!ok) break;
                // Orders the epilogue's TMEM reads (published by its arrive) before the MMAs that
                // overwrite the buffer.
                tc_fence_after_sync();
                FG_PROF_T0(tw2);
                ok = __all_sync(0xffffffffu, mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3));
                FG_PROF_ADD(prof_full, tw2);
                if (!ok) break;
                // My turn: the other warp has handed block j - 1 to the tensor core.
                FG_PROF_T0(tw3);
                {
                    uint32_t spins = 0;
                    const uint64_t t0 = global_timer_ns();
                    while (*issued_blocks != j) {
                        if ((++spins & 0xffu) == 0u) {
                            if (*abort_flag) { ok = false; break; }
                            if (global_timer_ns() - t0 > 2000000000ull) {
                                *abort_flag = 1u;
                                if (p.status) atomicCAS(p.status, 0u, (1u << 16) | 6u);
                                ok = false;
                                break;
                            }
                        }
                    }
                }
                FG_PROF_ADD(prof_turn, tw3);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (elect_one()) {
                    const uint32_t a_addr = smem_u32(smem + stage * C::STAGE_BYTES);
                    const uint64_t a_desc = umma_desc_k_sw128(a_addr);
                    const uint64_t b_desc = umma_desc_k_sw128(a_addr + C::A_BYTES);
                    const uint32_t d_tmem = tmem_base + me * BN;
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
                        umma_f8f6f4(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, k == 0 ? 0u : 1u);
                    *issued_blocks = j + 1u;
                    umma_commit(&tmem_full[me]);
                    umma_commit(&empty_bar[stage]);
                }
                __syncwarp();
#ifdef FG_GEMM_PROFILE
                ++prof_blocks;
#endif
            }
        }
#ifdef FG_GEMM_PROFILE
        if (lane == 0 && me == 0) {
            FG_PROF_OUT(1, prof_tmem);
            FG_PROF_OUT(2, prof_full);
            FG_PROF_OUT(3, clock64() - prof_start);
            FG_PROF_OUT(4, 2 * prof_blocks);
            FG_PROF_OUT(11, prof_turn);
        }
#endif
    } else if (warp == 1) {
        // ------------------------------- MMA issuer ---------------------------------------
        // The whole warp walks the loop (so that addresses and descriptors stay warp-uniform) and
        // one elected lane issues.  The tensor core queues only about six MMAs, i.e. one and a
        // half K blocks, so everything this warp does between two K blocks is on the critical
        // path: the state of the next K block's barriers is therefore probed (non-blocking)
        // before the current block's MMAs are issued, and the blocking wait is only the fallback.
        if (cta_rank == 0) {
            constexpr uint32_t idesc = OPK == 1 ? umma_idesc_s8_s32(BLOCK_M, BN)
                                       : OPK >= 2 ? umma_idesc_16bit_f32(BLOCK_M, BN, OPK == 2)
                                                  : umma_idesc_e4m3_f32(PAIR ? 2 * BLOCK_M : BLOCK_M, BN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t acc_iter = 0;
            bool ok = true;
            bool full_ready = false, tmem_ready = false;  // probed ahead for (stage, phase) / acc_iter
            FG_PROF_DECL(prof_tmem);
            FG_PROF_DECL(prof_full);
            FG_PROF_DECL(prof_blocks);
            FG_PROF_T0(prof_start);
            auto issue_block = [&](uint32_t a_addr, uint32_t d_tmem, auto zero_first) {
                const uint64_t a_desc = umma_desc_k_sw128(a_addr);
                const uint64_t b_desc = umma_desc_k_sw128(a_addr + C::A_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    // advancing K by 32 bytes inside the swizzle row: +2 in 16-byte units
                    const uint32_t accumulate = (decltype(zero_first)::value && k == 0) ? 0u : 1u;
                    if constexpr (PAIR)
                        umma_f8f6f4_2cta(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, accumulate);
                    else if constexpr (INT8)
                        umma_i8(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, accumulate);
                    else if constexpr (OPK >= 2)
                        umma_f16(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, accumulate);
                    else
                        umma_f8f6f4(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc, accumulate);
                }
            };
            for (int t = tile_first; t < num_tiles && ok; t += tile_step) {
                const TileCoord tc = tile_coord(t, num_m, num_n);
                const int expert = p.grouped ? p.expert_ids[tc.m_blk] : 0;
                if (expert < 0) continue;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const uint32_t buf = acc_iter & 1u;
                    const bool new_acc = BLOCK_SCALED || kb == kb_begin;
                    if (new_acc) {
                        FG_PROF_T0(tw);
                        ok = __all_sync(0xffffffffu, tmem_ready || mbar_wait(&tmem_empty[buf], ((acc_iter >> 1) & 1u) ^ 1u,
                                                                             abort_flag, p.status, 2));
                        FG_PROF_ADD(prof_tmem, tw);
                        if (!ok) break;
                        // Orders the epilogue's TMEM reads (published by its arrive) before the MMAs
                        // that overwrite the buffer.  The operand tiles need no fence: TMA writes
                        // and MMA reads are async-proxy accesses ordered by the full barrier.
                        tc_fence_after_sync();
                    }
                    FG_PROF_T0(tw2);
                    ok = __all_sync(0xffffffffu, full_ready || mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3));
                    FG_PROF_ADD(prof_full, tw2);
#ifdef FG_GEMM_PROFILE
                    ++prof_blocks;
#endif
                    if (!ok) break;
                    const uint32_t a_addr = smem_u32(smem + stage * C::STAGE_BYTES);
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    uint64_t* this_empty = &empty_bar[stage];
                    const bool last = BLOCK_SCALED || kb == kb_end - 1;
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    // Probe the next K block's barriers now; the answers arrive while the MMAs issue.
                    full_ready = mbar_test_wait(&full_bar[stage], phase);
                    if (last) {
                        const uint32_t nxt = acc_iter + 1u;
                        tmem_ready = mbar_test_wait(&tmem_empty[nxt & 1u], ((nxt >> 1) & 1u) ^ 1u);
                    }
                    if (elect_one()) {
                        if (new_acc) issue_block(a_addr, d_tmem, std::true_type{});
                        else issue_block(a_addr, d_tmem, std::false_type{});
                        if constexpr (PAIR) umma_commit_2cta(this_empty, 3); else umma_commit(this_empty);
                        if (last) {
                            if constexpr (PAIR) umma_commit_2cta(&tmem_full[buf], 3); else umma_commit(&tmem_full[buf]);
                        }
                    }
                    __syncwarp();
                    if (last) ++acc_iter;
                }
            }
#ifdef FG_GEMM_PROFILE
            if (lane == 0) {
                FG_PROF_OUT(1, prof_tmem);
                FG_PROF_OUT(2, prof_full);
                FG_PROF_OUT(3, clock64() - prof_start);
                FG_PROF_OUT(4, prof_blocks);
            }
#endif
        }
      }
    } else {
        // ------------------------------- epilogue -----------------------------------------
        if constexpr (C::REBALANCE_REGS) setmaxnreg_inc<C::REGS_EPILOGUE>();
        const int ew = warp - C::FIRST_EPI_WARP;
        const int quad = warp & 3;                  // TMEM lanes this warp may touch: [32*quad, +32)
        const int half = C::EPI_WARPS == 8 ? ew / 4 : 0;
        const int r_in_tile = quad * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
        uint8_t* epi_stage = epi_stage_base + ew * C::EPI_STAGE_BYTES;
        uint32_t acc_iter = 0;
        bool ok = true;
        FG_PROF_DECL(prof_epi_wait);
        FG_PROF_DECL(prof_epi_tail);
        FG_PROF_DECL(prof_epi_ld);
        FG_PROF_DECL(prof_epi_fma);
        FG_PROF_T0(prof_epi_start);
        uint32_t park_iter = 0;  // ASTORE: tiles parked so far

        for (int t = tile_first; t < num_tiles && ok; t += tile_step) {
            const TileCoord tc = tile_coord(t, num_m, num_n);
            const int expert = p.grouped ? p.expert_ids[tc.m_blk] : 0;
            const int m0 = tc.m_blk * a_rows_step + (int)cta_rank * BLOCK_M;
            const int n0 = tc.n_blk * OUT_TILE_N;
            const int64_t row = (int64_t)m0 + r_in_tile;  // row of A (sorted row when grouped)

            // Where this thread's row goes, and whether it is written at all.
            bool row_ok;
            int64_t out_row = row;
            float weight = 1.0f;
            if (p.grouped) {
                row_ok = r_in_tile < p.block_rows;
                if (row_ok && (p.scatter || p.mul_weight)) {
                    const int32_t sid = p.sorted_ids[row];
                    const bool real = sid >= 0 && sid < p.numel;
                    if (p.scatter) {
                        row_ok = real;
                        out_row = sid;
                    }
                    if (p.mul_weight && real) weight = load_as_float(p.topk_w, p.topk_w_dtype, (int64_t)sid * p.topk_w_stride);
                }
            } else {
                row_ok = row < p.M;
            }
            const int esz = out_elem_size(p.out_dtype);
            uint8_t* out_base = reinterpret_cast<uint8_t*>(p.c);
            if (p.n_peers > 0 && p.grouped && p.scatter && row_ok) {
                const int32_t* d = p.dest + out_row * p.dest_stride;
                const int32_t home = d[1];
                out_row = d[0];
                row_ok = home >= 0 && home < p.n_peers && out_row >= 0 && out_row < p.peer_rows;
                if (!row_ok && p.status) atomicCAS(p.status, 0u, (2u << 16) | 2u);
                out_base = reinterpret_cast<uint8_t*>(p.peer_out[row_ok ? home : 0]);
                if (!row_ok) out_row = 0;
            }
            uint8_t* out_ptr = out_base + out_row * p.ld_c * esz;
            // column of output chunk c (32 wide) handled by this thread
            const int out_col_base = n0 + (FUSE_SILU ? 64 * half : 128 * half);
            constexpr int OUT_CHUNKS = FUSE_SILU ? 2 : C::COLS / 32;

            if (expert < 0) {
                // Block of an expert that is not on this rank: the rows are defined to be zero.
                if (row_ok) {
                    float z[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) z[i] = 0.0f;
#pragma unroll
                    for (int c = 0; c < OUT_CHUNKS; ++c) {
                        const int col = out_col_base + 32 * c;
                        const int nc = min(32, p.n_out - col);
                        if (nc > 0) store_chunk(out_ptr, col, z, nc, p.out_dtype, p.c_vec_ok);
                    }
                }
                continue;
            }
            const int64_t srow = p.grouped ? row : (row < p.M ? row : p.M - 1);  // row used for scale loads

            if constexpr (!BLOCK_SCALED) {
                const uint32_t buf = acc_iter & 1u;
                ok = mbar_wait(&tmem_full[buf], (acc_iter >> 1) & 1u, abort_flag, p.status, 4);
                if (!ok) break;
                tc_fence_after_sync();
                const float sa = p.sa_mode == FG_SCALE_VECTOR ? p.sa[srow] : p.sa[0];
                const float* sbp = p.sb + (p.sb_mode == FG_SCALE_VECTOR ? (int64_t)expert * p.sb_stride_e : (int64_t)expert * (p.grouped ? 1 : 0));
                const uint32_t tbuf = lane_addr + buf * BN;
#pragma unroll
                for (int c = 0; c < OUT_CHUNKS; ++c) {
                    const int col = out_col_base + 32 * c;
                    uint32_t raw[32];
                    float v[32];
                    if constexpr (FUSE_SILU) {
                        uint32_t raw_up[32];
                        tmem_ld_32x32b_x32(tbuf + 64 * half + 32 * c, raw);
                        tmem_ld_32x32b_x32(tbuf + BN / 2 + 64 * half + 32 * c, raw_up);
                        tmem_ld_wait();
                        const int up_off = p.N / 2;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = min(col + i, p.n_out - 1);
                            const float sg = p.sb_mode == FG_SCALE_VECTOR ? __ldg(sbp + n) : sbp[0];
                            const float su = p.sb_mode == FG_SCALE_VECTOR ? __ldg(sbp + up_off + n) : sbp[0];
                            const float g = acc_f(raw[i]) * sa * sg;
                            const float u = acc_f(raw_up[i]) * sa * su;
                            v[i] = silu_mul(g, u);
                        }
                    } else if constexpr (SPLITK) {
                        tmem_ld_32x32b_x32(tbuf + 128 * half + 32 * c, raw);
                        tmem_ld_wait();
                        float* dst = reinterpret_cast<float*>(smem) + (size_t)r_in_tile * (BN + 4) + 128 * half + 32 * c;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<uint4*>(dst)[i] = make_uint4(raw[4 * i], raw[4 * i + 1], raw[4 * i + 2], raw[4 * i + 3]);
                    } else {
                        tmem_ld_32x32b_x32(tbuf + 128 * half + 32 * c, raw);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int n = min(col + i, p.n_out - 1);
                            const float sb = p.sb_mode == FG_SCALE_VECTOR ? __ldg(sbp + n) : sbp[0];
                            float x = sb * (sa * acc_f(raw[i]));
                            x *= weight;
                            if (p.bias) {
                                const float b = load_as_float(p.bias, p.bias_dtype, n + (int64_t)expert * p.bias_stride_e);
                                x = p.bias_after_round ? round_through(x, p.out_dtype) + b : x + b;
                            }
                            v[i] = x;
                        }
                    }
                    if constexpr (!SPLITK) {
                        const int nc = min(32, p.n_out - col);
                        if (nc == 32 && p.c_vec_ok && esz == 2)
                            store_chunk_coalesced(epi_stage, lane, v, out_ptr, row_ok, col, p.out_dtype);
                        else if (row_ok && nc > 0)
                            store_chunk(out_ptr, col, v, nc, p.out_dtype, p.c_vec_ok);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0u));
                    else mbar_arrive(&tmem_empty[buf]);
                }
                ++acc_iter;
            } else {
                // COLS fp32 accumulators per thread, kept as packed pairs for FFMA2.
                uint64_t acc[C::COLS / 2];
#pragma unroll
                for (int i = 0; i < C::COLS / 2; ++i) acc[i] = 0ull;
                // Block row of Bs for this thread's columns (two of them with fused SiLU).
                const float* bs_e = p.sb + (int64_t)expert * p.bs_stride_e;
                int nb0, nb1;
                if constexpr (FUSE_SILU) {
                    nb0 = (n0 + 64 * half) / 128;
                    nb1 = (p.N / 2 + n0 + 64 * half) / 128;
                } else {
                    nb0 = nb1 = (n0 + 128 * half) / 128;
                }
                const int max_nb = (p.N + 127) / 128 - 1;
                nb0 = min(nb0, max_nb);
                nb1 = min(nb1, max_nb);
                const float* as_row = p.sa + srow * p.ld_as;
                const float* bs0 = bs_e + nb0 * p.bs_stride_n;
                const float* bs1 = bs_e + nb1 * p.bs_stride_n;
                auto chunk_col = [&](int c) -> uint32_t {
                    if constexpr (FUSE_SILU) return (uint32_t)((c < 2 ? 0 : BN / 2) + 64 * half + 32 * (c & 1));
                    else return (uint32_t)(128 * half + 32 * c);
                };
                // Wide tiles issued by two warps (DUAL): scales of four K blocks at a time, fetched one
                // group ahead (a group lasts ~3000 cycles, so the loads are long complete when their
                // turn comes): 16-byte loads where the K-block scales of a row are contiguous and
                // aligned, four scalar loads otherwise.  Everywhere else (narrow tiles, split-K
                // slices of a handful of K blocks) one K block ahead: measured 3-4 us faster there
                // at decode sizes than the groups.
                constexpr bool SCALE_GROUPS = DUAL;
                const bool as_vec = p.as_stride_k == 1 && ((reinterpret_cast<uintptr_t>(as_row) & 15) == 0);
                const bool bs_vec = p.bs_stride_k == 1 && ((reinterpret_cast<uintptr_t>(bs0) & 15) == 0) &&
                                    ((reinterpret_cast<uintptr_t>(bs1) & 15) == 0);
                auto load4 = [&](const float* base, int64_t stride, bool vec, int kb0, bool ldg) -> float4 {
                    if (vec && (kb0 & 3) == 0 && kb0 + 4 <= num_k_blocks) {
                        return ldg ? __ldg(reinterpret_cast<const float4*>(base + kb0))
                                   : *reinterpret_cast<const float4*>(base + kb0);
                    }
                    float v[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int kk = min(kb0 + i, num_k_blocks - 1);
                        v[i] = ldg ? __ldg(base + (int64_t)kk * stride) : base[(int64_t)kk * stride];
                    }
                    return make_float4(v[0], v[1], v[2], v[3]);
                };
                float4 a_nx = make_float4(0.f, 0.f, 0.f, 0.f), b0_nx = a_nx, b1_nx = a_nx;
                float as_next = 0.f, b0_next = 0.f, b1_next = 0.f;
                if constexpr (SCALE_GROUPS) {
                    a_nx = load4(as_row, p.as_stride_k, as_vec, kb_begin, false);
                    b0_nx = load4(bs0, p.bs_stride_k, bs_vec, kb_begin, true);
                    b1_nx = FUSE_SILU ? load4(bs1, p.bs_stride_k, bs_vec, kb_begin, true) : b0_nx;
                } else {
                    as_next = as_row[(int64_t)kb_begin * p.as_stride_k];
                    b0_next = __ldg(bs0 + (int64_t)kb_begin * p.bs_stride_k);
                    if constexpr (FUSE_SILU) b1_next = __ldg(bs1 + (int64_t)kb_begin * p.bs_stride_k);
                }
                float g0[4] = {0.f, 0.f, 0.f, 0.f}, g1[4] = {0.f, 0.f, 0.f, 0.f};  // products of the current group
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    const int in_group = (kb - kb_begin) & 3;
                    float sc0f, sc1f;
                    if constexpr (!SCALE_GROUPS) {
                        sc0f = as_next * b0_next;
                        sc1f = FUSE_SILU ? as_next * b1_next : sc0f;
                        if (kb + 1 < kb_end) {  // next block's scales travel while this block is folded in
                            as_next = as_row[(int64_t)(kb + 1) * p.as_stride_k];
                            b0_next = __ldg(bs0 + (int64_t)(kb + 1) * p.bs_stride_k);
                            if constexpr (FUSE_SILU) b1_next = __ldg(bs1 + (int64_t)(kb + 1) * p.bs_stride_k);
                        }
                    } else {
                        if (in_group == 0) {
                            g0[0] = a_nx.x * b0_nx.x; g0[1] = a_nx.y * b0_nx.y; g0[2] = a_nx.z * b0_nx.z; g0[3] = a_nx.w * b0_nx.w;
                            if constexpr (FUSE_SILU) {
                                g1[0] = a_nx.x * b1_nx.x; g1[1] = a_nx.y * b1_nx.y; g1[2] = a_nx.z * b1_nx.z; g1[3] = a_nx.w * b1_nx.w;
                            }
                            if (kb + 4 < kb_end) {
                                a_nx = load4(as_row, p.as_stride_k, as_vec, kb + 4, false);
                                b0_nx = load4(bs0, p.bs_stride_k, bs_vec, kb + 4, true);
                                if constexpr (FUSE_SILU) b1_nx = load4(bs1, p.bs_stride_k, bs_vec, kb + 4, true);
                            }
                        }
                        sc0f = in_group == 0 ? g0[0] : in_group == 1 ? g0[1] : in_group == 2 ? g0[2] : g0[3];
                        sc1f = !FUSE_SILU ? sc0f
                               : in_group == 0 ? g1[0] : in_group == 1 ? g1[1] : in_group == 2 ? g1[2] : g1[3];
                    }
                    const uint64_t sc0 = pack_f32x2(sc0f, sc0f), sc1 = pack_f32x2(sc1f, sc1f);
                    const uint32_t buf = acc_iter & 1u;
                    FG_PROF_T0(tw);
                    ok = mbar_wait(&tmem_full[buf], (acc_iter >> 1) & 1u, abort_flag, p.status, 5);
                    FG_PROF_ADD(prof_epi_wait, tw);
                    if (!ok) break;
                    FG_PROF_T0(t_ld);
                    tc_fence_after_sync();
                    const uint32_t tbuf = lane_addr + buf * BN;
                    auto release = [&]() {
                        // Every column of this buffer is in registers: hand it back to the MMA warp
                        // before the last part is folded.
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (PAIR) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[buf]), 0u));
                            else mbar_arrive(&tmem_empty[buf]);
                        }
                        FG_PROF_ADD(prof_epi_ld, t_ld);
                    };
                    if constexpr (C::COLS == 128) {
                        // Four 32-column loads through two register sets, software-pipelined: the
                        // third and fourth load travel while the first two sets are folded, and the
                        // buffer goes back to the MMA warp before the last 32 packed FMAs.  Measured
                        // on the bare loop: 286 cycles per K block against 405 for two rounds of
                        // (64-column load, wait, fold); the 64 packed FMAs of a thread alone take
                        // 256 cycles per K block and scheduler, the MMAs of a K block 525.
                        uint32_t v0[32], v1[32];
                        tmem_ld_32x32b_x32(tbuf + chunk_col(0), v0);
                        tmem_ld_32x32b_x32(tbuf + chunk_col(1), v1);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) ffma2(acc[i], v0[2 * i], v0[2 * i + 1], sc0);
                        tmem_ld_32x32b_x32(tbuf + chunk_col(2), v0);
#pragma unroll
                        for (int i = 0; i < 16; ++i) ffma2(acc[16 + i], v1[2 * i], v1[2 * i + 1], sc0);
                        tmem_ld_32x32b_x32(tbuf + chunk_col(3), v1);
                        tmem_ld_wait();
                        release();
                        FG_PROF_T0(t_f);
#pragma unroll
                        for (int i = 0; i < 16; ++i) ffma2(acc[32 + i], v0[2 * i], v0[2 * i + 1], sc1);
#pragma unroll
                        for (int i = 0; i < 16; ++i) ffma2(acc[48 + i], v1[2 * i], v1[2 * i + 1], sc1);
                        FG_PROF_ADD(prof_epi_fma, t_f);
                    } else if constexpr (C::COLS == 64) {
                        uint32_t raw[64];
                        tmem_ld_32x32b_x64(tbuf + chunk_col(0), raw);
                        tmem_ld_wait();
                        release();
#pragma unroll
                        for (int i = 0; i < 32; ++i) ffma2(acc[i], raw[2 * i], raw[2 * i + 1], sc0);
                    } else {
                        uint32_t raw[32];
                        tmem_ld_32x32b_x32(tbuf + chunk_col(0), raw);
                        tmem_ld_wait();
                        release();
#pragma unroll
                        for (int i = 0; i < 16; ++i) ffma2(acc[i], raw[2 * i], raw[2 * i + 1], sc0);
                    }
                    ++acc_iter;
                }
                if (!ok) break;
                FG_PROF_T0(t_tail);
                if constexpr (ASTORE) {
                    // Park the converted tile for the store warp: rows of OUT_TILE_N 16-bit values, the
                    // 16-byte pieces of a row XOR-swizzled by (row & 7) so that the 32 rows a warp writes
                    // at once and the row the store warp reads at once both spread over all banks.
                    ok = mbar_wait(park_free, (park_iter & 1u) ^ 1u, abort_flag, p.status, 7);
                    if (!ok) break;
                    constexpr int ROW_BYTES = OUT_TILE_N * 2;
                    uint8_t* prow = park_tile + r_in_tile * ROW_BYTES;
#pragma unroll
                    for (int c = 0; c < OUT_CHUNKS; ++c) {
                        uint32_t w[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint64_t a = acc[16 * c + i];
                            float lo, hi;
                            if constexpr (FUSE_SILU) {
                                const uint64_t u = acc[32 + 16 * c + i];
                                lo = silu_mul(f32x2_lo(a), f32x2_lo(u));
                                hi = silu_mul(f32x2_hi(a), f32x2_hi(u));
                            } else {
                                lo = f32x2_lo(a) * weight;
                                hi = f32x2_hi(a) * weight;
                            }
                            if (p.out_dtype == FG_DTYPE_BF16) {
                                __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
                                w[i] = *reinterpret_cast<uint32_t*>(&h2);
                            } else {
                                __half2 h2 = __floats2half2_rn(lo, hi);
                                w[i] = *reinterpret_cast<uint32_t*>(&h2);
                            }
                        }
                        const int piece0 = ((FUSE_SILU ? 64 * half : 128 * half) + 32 * c) / 8;
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            *reinterpret_cast<uint4*>(prow + (((piece0 + k) ^ (r_in_tile & 7)) << 4)) =
                                make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
                    }
                    if (half == 0) park_rows[r_in_tile] = row_ok ? reinterpret_cast<unsigned long long>(out_ptr) : 0ull;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(park_full);
                    ++park_iter;
                } else if constexpr (SPLITK) {
                    float* dst = reinterpret_cast<float*>(smem) + (size_t)r_in_tile * (BN + 4) + 128 * half;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        reinterpret_cast<uint4*>(dst)[i] =
                            make_uint4((uint32_t)(acc[2 * i] & 0xffffffffull), (uint32_t)(acc[2 * i] >> 32),
                                       (uint32_t)(acc[2 * i + 1] & 0xffffffffull), (uint32_t)(acc[2 * i + 1] >> 32));
                } else
#pragma unroll
                for (int c = 0; c < OUT_CHUNKS; ++c) {
                    const int col = out_col_base + 32 * c;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const uint64_t a = acc[16 * c + i];
                        if constexpr (FUSE_SILU) {
                            const uint64_t u = acc[32 + 16 * c + i];
                            v[2 * i] = silu_mul(f32x2_lo(a), f32x2_lo(u));
                            v[2 * i + 1] = silu_mul(f32x2_hi(a), f32x2_hi(u));
                        } else {
                            v[2 * i] = f32x2_lo(a) * weight;
                            v[2 * i + 1] = f32x2_hi(a) * weight;
                        }
                    }
                    const int nc = min(32, p.n_out - col);
                    if (nc == 32 && p.c_vec_ok && esz == 2)
                        store_chunk_coalesced(epi_stage, lane, v, out_ptr, row_ok, col, p.out_dtype);
                    else if (row_ok && nc > 0)
                        store_chunk(out_ptr, col, v, nc, p.out_dtype, p.c_vec_ok);
                }
                FG_PROF_ADD(prof_epi_tail, t_tail);
            }
        }
#ifdef FG_GEMM_PROFILE
        if (ew == 0 && lane == 0) {
            FG_PROF_OUT(5, prof_epi_wait);
            FG_PROF_OUT(6, prof_epi_tail);
            FG_PROF_OUT(7, clock64() - prof_epi_start);
            FG_PROF_OUT(8, prof_epi_ld);
            FG_PROF_OUT(9, prof_epi_fma);
        }
#endif
    }

    if constexpr (SPLITK) {
        // ------------------------- cluster reduction of the K slices ---------------------------
        // Every thread of every CTA of the cluster reaches both syncs, also after a failed wait.
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();  // all partial tiles are in shared memory
        if (warp >= C::FIRST_EPI_WARP && tile_first < num_tiles) {
            const TileCoord tc = tile_coord(tile_first, num_m, num_n);
            const int n0 = tc.n_blk * BN;
            const int m0 = tc.m_blk * BLOCK_M;
            const int rows = (int)min((int64_t)BLOCK_M, p.M - m0);
            const int width = BN / k_slices;            // columns this CTA finishes (multiple of 4)
            const int c_first = (int)cluster.block_rank() * width;
            const int vec_per_row = width / 4;
            const int esz = out_elem_size(p.out_dtype);
            const float* part[8];
            for (int q = 0; q < k_slices; ++q)
                part[q] = cluster.map_shared_rank(reinterpret_cast<float*>(smem), q);
            const int n_epi = C::EPI_WARPS * 32;
            for (int idx = threadIdx.x - C::FIRST_EPI_WARP * 32; idx < rows * vec_per_row; idx += n_epi) {
                const int r = idx / vec_per_row, c = c_first + (idx % vec_per_row) * 4;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int q = 0; q < k_slices; ++q) {
                    const float4 v = *reinterpret_cast<const float4*>(part[q] + (size_t)r * (BN + 4) + c);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                float o[4] = {sum.x, sum.y, sum.z, sum.w};
                const int64_t row = (int64_t)m0 + r;
                if constexpr (!BLOCK_SCALED) {
                    const float sa = p.sa_mode == FG_SCALE_VECTOR ? p.sa[row] : p.sa[0];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = min(n0 + c + i, p.n_out - 1);
                        const float sb = p.sb_mode == FG_SCALE_VECTOR ? __ldg(p.sb + n) : p.sb[0];
                        float x = sb * (sa * o[i]);
                        if (p.bias) {
                            const float b = load_as_float(p.bias, p.bias_dtype, n);
                            x = p.bias_after_round ? round_through(x, p.out_dtype) + b : x + b;
                        }
                        o[i] = x;
                    }
                }
                uint8_t* out = reinterpret_cast<uint8_t*>(p.c) + (row * p.ld_c + n0 + c) * esz;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (n0 + c + i >= p.n_out) break;
                    if (p.out_dtype == FG_DTYPE_BF16) reinterpret_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(o[i]);
                    else if (p.out_dtype == FG_DTYPE_F16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(o[i]);
                    else if (p.out_dtype == FG_DTYPE_E4M3)
                        out[i] = (uint8_t)(__nv_cvt_float2_to_fp8x2(make_float2(o[i], 0.0f), __NV_SATFINITE, __NV_E4M3) & 0xffu);
                    else reinterpret_cast<float*>(out)[i] = o[i];
                }
            }
        }
        cluster.sync();  // nobody leaves while a peer may still read its partial tile
    }

    // ------------------------------- teardown ---------------------------------------------
    tc_fence_before_sync();
    if constexpr (PAIR) cluster_sync_all();  // neither CTA leaves while the pair's MMAs may touch it
    else __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Byte tensor [d2][d1][d0] with d0 contiguous; box = 128 x box_rows x 1, 128-byte swizzle.
int make_map(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1,
             uint64_t stride2, uint32_t box_rows, int rank) {
    EncodeTiledFn fn = get_encode_fn();
    FG_REQUIRE(fn != nullptr, FG_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {128, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FG_REQUIRE(r == CUDA_SUCCESS, FG_ERR_CUDA,
               "cuTensorMapEncodeTiled failed (%d): base %p dims %llu x %llu x %llu strides %llu, %llu box rows %u",
               (int)r, base, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
               (unsigned long long)stride1, (unsigned long long)stride2, box_rows);
    return FG_OK;
}

// How many clusters of `slices` CTAs of the split-K kernel fit on the device at once (cached).
template <int BN, bool BS>
int max_resident_clusters(int slices) {
    static int table[64][9];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    int* cache = table[fg_device_index()];
    if (cache[slices]) return cache[slices];
    using C = Cfg<BN, false>;
    auto kernel = gemm_fp8_kernel<BN, BS, false, false, true>;
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(slices * 64), 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)slices;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        n = 1;
    }
    cache[slices] = n;
    return n;
}

template <int BN, bool BS>
int launch_splitk(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int tiles, int slices,
                  cudaStream_t st) {
    using C = Cfg<BN, false>;
    auto kernel = gemm_fp8_kernel<BN, BS, false, false, true>;
    static bool attr_done[64];
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        bool& done = attr_done[fg_device_index()];
        if (!done) {
            FG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
            done = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(tiles * slices), 1, 1);
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)slices;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    FG_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
    fg_count_launch(1);
    return FG_OK;
}

// CTA-pair kernel: clusters of two, one cluster per 256 x 256 tile, persistent over the tiles.
// Dense scales only: with block scales the accumulator of every K block has to make the round
// trip MMA -> both CTAs' epilogues -> MMA through cluster-wide barriers, and that latency costs
// more than the halved B traffic saves (measured: about half the single-CTA throughput).
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int pair_tiles, cudaStream_t st) {
    using C = Cfg<256, false, true>;
    auto kernel = gemm_fp8_kernel<256, false, false, false, false, true>;
    static int max_clusters_dev[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    int& max_clusters = max_clusters_dev[fg_device_index()];
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(C::THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (!max_clusters) {
        FG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        cfg.gridDim = dim3((unsigned)(2 * (fg_num_sms() / 2)), 1, 1);
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 1;
        }
        max_clusters = n < fg_num_sms() / 2 ? n : fg_num_sms() / 2;
    }
    const int clusters = pair_tiles < max_clusters ? pair_tiles : max_clusters;
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    FG_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, p));
    fg_count_launch(1);
    return FG_OK;
}

// FG_GEMM_PAIR=0 keeps every dense product on the single-CTA kernels (for comparison runs).
bool pair_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("FG_GEMM_PAIR");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

template <int BN, bool BS, bool SILU, bool SMALL_A = false, bool ASTORE = false, int OPK = 0>
int launch_inst(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int max_tiles, cudaStream_t st) {
    using C = Cfg<BN, SMALL_A, false, ASTORE>;
    auto kernel = gemm_fp8_kernel<BN, BS, SILU, SMALL_A, false, false, ASTORE, OPK>;
    static bool attr_done[64];
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        bool& done = attr_done[fg_device_index()];
        if (!done) {
            FG_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
            done = true;
        }
    }
    int grid = fg_num_sms();
    if (max_tiles < grid) grid = max_tiles;
    if (grid < 1) grid = 1;
    kernel<<<grid, C::THREADS, C::SMEM_BYTES, st>>>(ta, tb, p);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int launch_gemm(GemmParams& p, const void* a, int64_t a_rows, int64_t ld_a, const void* b, int num_experts,
                int64_t ld_b, bool block_scaled, bool fuse_silu, cudaStream_t st) {
    FG_REQUIRE(p.K > 0 && p.K % 16 == 0, FG_ERR_UNSUPPORTED, "K = %d must be a positive multiple of 16", p.K);
    FG_REQUIRE((uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 && ld_a % 16 == 0 && ld_b % 16 == 0,
               FG_ERR_UNSUPPORTED, "a and b must be 16-byte aligned with row strides that are multiples of 16 bytes");
    FG_REQUIRE(ld_a >= p.K && ld_b >= p.K, FG_ERR_INVALID_ARGUMENT, "row stride smaller than K");
    p.status = fg_status_word_device_ptr();
    const int esz = out_elem_size(p.out_dtype);
    p.c_vec_ok = ((uintptr_t)p.c % 16 == 0) && ((p.ld_c * esz) % 16 == 0);

    const int64_t m_tiles = p.grouped ? a_rows / p.block_rows : fg_cdiv(p.M, BLOCK_M);
    const int sms = fg_num_sms();
    // Tile width.  One K block costs a CTA about the same time whatever the width (an MMA with
    // M = 128 streams 128 rows of A however few columns it has), so the widest tile wins as long
    // as most SMs still get a tile; below that, narrower tiles buy CTAs.
    const int64_t enough = (int64_t)sms * 5 / 8;
    int bn;
    bool small_a = false;
    if (fuse_silu) {
        bn = m_tiles * fg_cdiv(p.n_out, 128) >= enough ? 256 : 128;
    } else if (m_tiles * fg_cdiv(p.n_out, 256) >= enough) {
        bn = 256;
    } else if (m_tiles * fg_cdiv(p.n_out, 128) >= enough || p.grouped) {
        bn = 128;
    } else if (m_tiles * fg_cdiv(p.n_out, 64) >= enough) {
        bn = 64;
    } else {
        bn = 32;
        small_a = p.M <= 32;
    }
    // Decode-sized M with fewer wide tiles than half the SMs: split K over a cluster instead of
    // narrowing the tile (a narrow tile still pays a full MMA per K step).
    int k_slices = 1;
    if (!p.grouped && !fuse_silu && m_tiles == 1) {
        const int wide = p.n_out >= 256 ? 256 : 128;
        const int64_t wide_tiles = fg_cdiv(p.n_out, wide);
        const int64_t nkb = fg_cdiv(p.K, BLOCK_K);
        for (int cand = 8; cand >= 2; cand /= 2) {
            const int64_t per = fg_cdiv(nkb, cand);
            const int resident = wide == 256
                ? (block_scaled ? max_resident_clusters<256, true>(cand) : max_resident_clusters<256, false>(cand))
                : (block_scaled ? max_resident_clusters<128, true>(cand) : max_resident_clusters<128, false>(cand));
            if (wide_tiles <= resident && per >= 2 && (cand - 1) * per < nkb) {
                k_slices = cand;
                bn = wide;
                small_a = false;
                break;
            }
        }
    }
    p.a_box_rows = BLOCK_M;
    if (!p.grouped && p.M < BLOCK_M) p.a_box_rows = (int)((p.M + 7) / 8 * 8);
    // Large dense products: a pair of CTAs per 256 x 256 tile (a third less L2 and shared-memory
    // traffic per flop: +4-5 % under the power cap) once there are at least three waves of such
    // tiles; with fewer, the coarser tiles lose more to the ragged last wave than they gain.
    const int64_t pair_tiles = fg_cdiv(p.M, 2 * BLOCK_M) * fg_cdiv(p.n_out, 256);
    const bool pair = !p.grouped && !fuse_silu && !block_scaled && bn == 256 && k_slices == 1 &&
                      pair_tiles >= 3 * (int64_t)(sms / 2) && pair_tiles < (1ll << 30) && pair_enabled();
    const int out_tile = fuse_silu ? bn / 2 : bn;
    const int64_t tiles = m_tiles * fg_cdiv(p.n_out, out_tile);
    FG_REQUIRE(tiles < (1ll << 31), FG_ERR_UNSUPPORTED, "too many tiles");
    if (tiles == 0) return FG_OK;

    CUtensorMap ta, tb;
    int rc = make_map(&ta, a, (uint64_t)p.K, (uint64_t)a_rows, 1, (uint64_t)ld_a, 0,
                      (uint32_t)(p.grouped ? p.block_rows : p.a_box_rows), 2);
    if (rc != FG_OK) return rc;
    rc = make_map(&tb, b, (uint64_t)p.K, (uint64_t)p.N, (uint64_t)num_experts, (uint64_t)ld_b,
                  (uint64_t)ld_b * (uint64_t)p.N, (uint32_t)((fuse_silu || pair) ? bn / 2 : bn), 3);
    if (rc != FG_OK) return rc;
    if (pair) return launch_pair(ta, tb, p, (int)pair_tiles, st);

    const int t = (int)tiles;
    if (p.int8) {
        FG_REQUIRE(!block_scaled && (bn == 256 || bn == 128) && k_slices == 1 && !pair, FG_ERR_UNSUPPORTED,
                   "int8 and 16-bit operands are built for the grouped expert GEMMs");
        auto by_kind = [&](auto bn_tag, auto silu_tag) -> int {
            constexpr int B = decltype(bn_tag)::value;
            constexpr bool S = decltype(silu_tag)::value;
            switch (p.int8) {
                case 1: return launch_inst<B, false, S, false, false, 1>(ta, tb, p, t, st);
                case 2: return launch_inst<B, false, S, false, false, 2>(ta, tb, p, t, st);
                default: return launch_inst<B, false, S, false, false, 3>(ta, tb, p, t, st);
            }
        };
        using I256 = std::integral_constant<int, 256>;
        using I128 = std::integral_constant<int, 128>;
        if (bn == 256) return fuse_silu ? by_kind(I256(), std::true_type()) : by_kind(I256(), std::false_type());
        return fuse_silu ? by_kind(I128(), std::true_type()) : by_kind(I128(), std::false_type());
    }
    if (k_slices > 1) {
        if (bn == 256) return block_scaled ? launch_splitk<256, true>(ta, tb, p, t, k_slices, st)
                                           : launch_splitk<256, false>(ta, tb, p, t, k_slices, st);
        return block_scaled ? launch_splitk<128, true>(ta, tb, p, t, k_slices, st)
                            : launch_splitk<128, false>(ta, tb, p, t, k_slices, st);
    }
    if (bn == 256) {
        // 16-bit outputs with 16-byte aligned rows: the tile is parked and written out by the store warp.
        // Not for a single row of tiles (M <= 128), where the job is to stream the weights and the
        // fourth ring stage is worth more than the store warp (measured 36 vs 42 us at N = 24576).
        const bool park = m_tiles > 1 && block_scaled && esz == 2 && p.c_vec_ok && p.n_out % 8 == 0;
        if (park) return fuse_silu ? launch_inst<256, true, true, false, true>(ta, tb, p, t, st)
                                   : launch_inst<256, true, false, false, true>(ta, tb, p, t, st);
        if (block_scaled) return fuse_silu ? launch_inst<256, true, true>(ta, tb, p, t, st)
                                           : launch_inst<256, true, false>(ta, tb, p, t, st);
        return fuse_silu ? launch_inst<256, false, true>(ta, tb, p, t, st)
                         : launch_inst<256, false, false>(ta, tb, p, t, st);
    }
    if (bn == 128) {
        if (block_scaled) return fuse_silu ? launch_inst<128, true, true>(ta, tb, p, t, st)
                                           : launch_inst<128, true, false>(ta, tb, p, t, st);
        return fuse_silu ? launch_inst<128, false, true>(ta, tb, p, t, st)
                         : launch_inst<128, false, false>(ta, tb, p, t, st);
    }
    if (bn == 64)
        return block_scaled ? launch_inst<64, true, false>(ta, tb, p, t, st)
                            : launch_inst<64, false, false>(ta, tb, p, t, st);
    if (small_a)
        return block_scaled ? launch_inst<32, true, false, true>(ta, tb, p, t, st)
                            : launch_inst<32, false, false, true>(ta, tb, p, t, st);
    return block_scaled ? launch_inst<32, true, false>(ta, tb, p, t, st)
                        : launch_inst<32, false, false>(ta, tb, p, t, st);
}

bool dtype_ok(int d) { return d == FG_DTYPE_BF16 || d == FG_DTYPE_F16 || d == FG_DTYPE_F32; }

// One thread waits, with the library's bounded wait, on an mbarrier phase that nothing completes.
__global__ void bounded_wait_selftest_kernel(unsigned int* status, uint64_t limit_ns, uint32_t site) {
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0u;
        fence_mbar_init();
        mbar_wait(&bar, 0u, &abort_flag, status, site, limit_ns);
    }
}

}  // namespace

extern "C" {

#ifdef FG_GEMM_PROFILE
// Development only: copies the stall counters of the last GEMM launch to the host.
int fg_debug_gemm_profile(long long* out, int n) {
    FG_CUDA(cudaDeviceSynchronize());
    FG_CUDA(cudaMemcpyFromSymbol(out, g_gemm_prof, sizeof(long long) * (size_t)(n < 3072 ? n : 3072)));
    return FG_OK;
}
#endif

int fg_selftest_bounded_wait(int64_t limit_ns, int site, void* stream) {
    FG_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ll, FG_ERR_INVALID_ARGUMENT,
               "limit_ns must be in (0, 100 ms]");
    bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(fg_status_word_device_ptr(), (uint64_t)limit_ns,
                                                                     (uint32_t)site);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_scaled_mm_fp8(void* c, const void* a, const void* b, const float* sa, const float* sb, const void* bias,
                     int64_t M, int64_t N, int64_t K, int64_t ld_a, int64_t ld_b, int64_t ld_c, int sa_mode,
                     int sb_mode, int out_dtype, int bias_after_round, void* stream) {
    FG_REQUIRE(M >= 0 && N >= 0 && K >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    if (M == 0 || N == 0) return FG_OK;
    FG_REQUIRE(c && a && b && sa && sb, FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE(dtype_ok(out_dtype) || out_dtype == FG_DTYPE_E4M3, FG_ERR_INVALID_ARGUMENT, "bad out_dtype %d", out_dtype);
    FG_REQUIRE((sa_mode == FG_SCALE_SCALAR || sa_mode == FG_SCALE_VECTOR) &&
                   (sb_mode == FG_SCALE_SCALAR || sb_mode == FG_SCALE_VECTOR),
               FG_ERR_INVALID_ARGUMENT, "scale modes must be scalar or vector");
    FG_REQUIRE(N < (1ll << 31) && K < (1ll << 31) && M < (1ll << 31), FG_ERR_UNSUPPORTED, "dimension too large");
    GemmParams p{};
    p.M = M; p.N = (int)N; p.K = (int)K; p.n_out = (int)N;
    p.c = c; p.ld_c = ld_c; p.out_dtype = out_dtype;
    p.sa = sa; p.sb = sb; p.bias = bias; p.sa_mode = sa_mode; p.sb_mode = sb_mode;
    p.bias_after_round = bias_after_round;
    p.bias_dtype = out_dtype == FG_DTYPE_E4M3 ? FG_DTYPE_F32 : out_dtype;  // fp32 bias only with the e4m3 output
    p.block_rows = BLOCK_M;
    return launch_gemm(p, a, M, ld_a, b, 1, ld_b, false, false, (cudaStream_t)stream);
}

int fg_block_scaled_mm_fp8(void* c, const void* a, const void* b, const float* a_s, const float* b_s, int64_t M,
                           int64_t N, int64_t K, int64_t ld_a, int64_t ld_b, int64_t ld_c, int64_t ld_as,
                           int64_t as_stride_k, int64_t bs_stride_n, int64_t bs_stride_k, int out_dtype,
                           void* stream) {
    FG_REQUIRE(M >= 0 && N >= 0 && K >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    if (M == 0 || N == 0) return FG_OK;
    FG_REQUIRE(c && a && b && a_s && b_s, FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE(dtype_ok(out_dtype), FG_ERR_INVALID_ARGUMENT, "bad out_dtype %d", out_dtype);
    FG_REQUIRE(N < (1ll << 31) && K < (1ll << 31) && M < (1ll << 31), FG_ERR_UNSUPPORTED, "dimension too large");
    GemmParams p{};
    p.M = M; p.N = (int)N; p.K = (int)K; p.n_out = (int)N;
    p.c = c; p.ld_c = ld_c; p.out_dtype = out_dtype;
    p.sa = a_s; p.sb = b_s; p.ld_as = ld_as; p.as_stride_k = as_stride_k;
    p.bs_stride_n = bs_stride_n; p.bs_stride_k = bs_stride_k;
    p.block_rows = BLOCK_M;
    return launch_gemm(p, a, M, ld_a, b, 1, ld_b, true, false, (cudaStream_t)stream);
}

int fg_moe_grouped_gemm_fp8(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                            const void* topk_weights, int topk_w_dtype, int64_t topk_w_stride,
                            const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_pad,
                            int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K, int64_t ld_a,
                            int64_t ld_c, int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                            int scatter, int mul_weight, int out_dtype, void* stream) {
    return fg_moe_grouped_gemm_fp8_peer(c, a, w, a_scale, w_scale, topk_weights, topk_w_dtype, topk_w_stride,
                                        sorted_ids, expert_ids, num_post_pad, max_rows, numel, num_experts, N, K,
                                        ld_a, ld_c, block_rows, scale_mode, a_scale_per_row, fuse_silu, scatter,
                                        mul_weight, out_dtype, nullptr, 0, nullptr, 0, 0, stream);
}

// Grouped GEMM with a per-row x per-column scale pair and an optional fp32 bias row per group (or one
// row for all groups): the device work of aten _scaled_grouped_mm, see fg_scaled_grouped_mm_fp8.
int fg_grouped_gemm_fp8_bias(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                             const float* bias, int64_t bias_stride_g, const int32_t* sorted_ids,
                             const int32_t* expert_ids, const int32_t* num_post_pad, int64_t max_rows, int64_t numel,
                             int num_groups, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c, int out_dtype,
                             void* stream) {
    FG_REQUIRE(max_rows >= 0 && N > 0 && K > 0 && num_groups > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(c && a && w && a_scale && w_scale && sorted_ids && expert_ids && num_post_pad, FG_ERR_INVALID_ARGUMENT,
               "null pointer");
    FG_REQUIRE(dtype_ok(out_dtype), FG_ERR_INVALID_ARGUMENT, "bad out_dtype %d", out_dtype);
    FG_REQUIRE(N < (1ll << 31) && K < (1ll << 31), FG_ERR_UNSUPPORTED, "dimension too large");
    if (max_rows == 0) return FG_OK;
    GemmParams p{};
    p.M = max_rows / BLOCK_M * BLOCK_M; p.N = (int)N; p.K = (int)K; p.n_out = (int)N;
    p.c = c; p.ld_c = ld_c; p.out_dtype = out_dtype;
    p.sa = a_scale; p.sb = w_scale; p.sa_mode = FG_SCALE_VECTOR; p.sb_mode = FG_SCALE_VECTOR; p.sb_stride_e = N;
    p.bias = bias; p.bias_dtype = FG_DTYPE_F32; p.bias_stride_e = bias_stride_g; p.bias_after_round = 0;
    p.grouped = 1; p.sorted_ids = sorted_ids; p.expert_ids = expert_ids; p.num_post_pad = num_post_pad;
    p.block_rows = BLOCK_M; p.numel = numel; p.scatter = 1; p.mul_weight = 0; p.topk_w_stride = 1;
    return launch_gemm(p, a, p.M, ld_a, w, num_groups, K, false, false, (cudaStream_t)stream);
}

static int grouped_gemm_common(int int8, void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                            const void* topk_weights, int topk_w_dtype, int64_t topk_w_stride,
                            const int32_t* sorted_ids,
                            const int32_t* expert_ids, const int32_t* num_post_pad, int64_t max_rows, int64_t numel,
                            int num_experts, int64_t N, int64_t K, int64_t ld_a, int64_t ld_c, int block_rows,
                            int scale_mode, int a_scale_per_row, int fuse_silu, int scatter, int mul_weight,
                            int out_dtype, const int32_t* dest, int64_t dest_stride, void* const* peer_out, int n_peers,
                            int64_t peer_rows, void* stream) {
    FG_REQUIRE(max_rows >= 0 && N > 0 && K > 0 && num_experts > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE((c || n_peers > 0) && a && w && a_scale && w_scale && sorted_ids && expert_ids && num_post_pad,
               FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE(n_peers >= 0 && n_peers <= 8 &&
                   (n_peers == 0 || (dest && peer_out && scatter && dest_stride >= 2 && peer_rows > 0)),
               FG_ERR_INVALID_ARGUMENT,
               "peer scatter needs 1..8 peers, scatter mode, a (slot, rank) table and the peers' row capacity");
    FG_REQUIRE(dtype_ok(out_dtype), FG_ERR_INVALID_ARGUMENT, "bad out_dtype %d", out_dtype);
    FG_REQUIRE(block_rows >= 8 && block_rows <= 128 && block_rows % 8 == 0, FG_ERR_UNSUPPORTED,
               "block_rows %d must be a multiple of 8 in [8, 128]", block_rows);
    FG_REQUIRE(!mul_weight || (topk_weights && dtype_ok(topk_w_dtype)), FG_ERR_INVALID_ARGUMENT,
               "mul_weight needs topk_weights");
    FG_REQUIRE(N < (1ll << 31) && K < (1ll << 31), FG_ERR_UNSUPPORTED, "dimension too large");
    FG_REQUIRE(!fuse_silu || N % 2 == 0, FG_ERR_INVALID_ARGUMENT, "fused SiLU needs an even N");
    const bool block = scale_mode == FG_SCALE_BLOCK;
    FG_REQUIRE(!(block && fuse_silu) || (N / 2) % 128 == 0, FG_ERR_UNSUPPORTED,
               "fused SiLU with block scales needs the intermediate size %lld to be a multiple of 128",
               (long long)(N / 2));
    if (max_rows == 0) return FG_OK;
    if (int8 >= 2) {  // 16-bit operands: the kernel counts K and the operand row strides in bytes
        FG_REQUIRE(!block && K % 8 == 0 && 2 * K < (1ll << 31), FG_ERR_UNSUPPORTED,
                   "16-bit operands take per-tensor or per-row x per-column scales and K a multiple of 8");
        K *= 2;
        ld_a *= 2;
    }
    GemmParams p{};
    p.M = max_rows / block_rows * block_rows; p.N = (int)N; p.K = (int)K; p.n_out = fuse_silu ? (int)(N / 2) : (int)N;
    p.c = c; p.ld_c = ld_c; p.out_dtype = out_dtype;
    p.sa = a_scale; p.sb = w_scale;
    if (block) {
        const int64_t kb = fg_cdiv(K, 128), nb = fg_cdiv(N, 128);
        p.ld_as = kb; p.as_stride_k = 1; p.bs_stride_k = 1; p.bs_stride_n = kb; p.bs_stride_e = kb * nb;
    } else {
        p.sa_mode = (scale_mode == FG_SCALE_VECTOR || a_scale_per_row) ? FG_SCALE_VECTOR : FG_SCALE_SCALAR;
        p.sb_mode = scale_mode == FG_SCALE_VECTOR ? FG_SCALE_VECTOR : FG_SCALE_SCALAR;
        p.sb_stride_e = N;
    }
    p.grouped = 1; p.int8 = int8; p.sorted_ids = sorted_ids; p.expert_ids = expert_ids; p.num_post_pad = num_post_pad;
    p.block_rows = block_rows; p.numel = numel; p.scatter = scatter; p.mul_weight = mul_weight;
    p.topk_w = topk_weights; p.topk_w_dtype = topk_w_dtype; p.topk_w_stride = topk_w_stride > 0 ? topk_w_stride : 1;
    p.dest = dest; p.dest_stride = dest_stride; p.n_peers = n_peers; p.peer_rows = peer_rows;
    for (int i = 0; i < n_peers; ++i) p.peer_out[i] = peer_out[i];
    if (n_peers > 0 && !c) p.c = peer_out[0];
    return launch_gemm(p, a, p.M, ld_a, w, num_experts, K, block, fuse_silu != 0, (cudaStream_t)stream);
}

int fg_moe_grouped_gemm_fp8_peer(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                                 const void* topk_weights, int topk_w_dtype, int64_t topk_w_stride,
                                 const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_pad,
                                 int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K, int64_t ld_a,
                                 int64_t ld_c, int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                                 int scatter, int mul_weight, int out_dtype, const int32_t* dest, int64_t dest_stride,
                                 void* const* peer_out, int n_peers, int64_t peer_rows, void* stream) {
    return grouped_gemm_common(0, c, a, w, a_scale, w_scale, topk_weights, topk_w_dtype, topk_w_stride, sorted_ids,
                               expert_ids, num_post_pad, max_rows, numel, num_experts, N, K, ld_a, ld_c, block_rows,
                               scale_mode, a_scale_per_row, fuse_silu, scatter, mul_weight, out_dtype, dest, dest_stride,
                               peer_out, n_peers, peer_rows, stream);
}

int fg_moe_grouped_gemm_16bit(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                              const void* topk_weights, int topk_w_dtype, int64_t topk_w_stride,
                              const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_pad,
                              int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K, int64_t ld_a,
                              int64_t ld_c, int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                              int scatter, int mul_weight, int operand_dtype, int out_dtype, void* stream) {
    FG_REQUIRE(operand_dtype == FG_DTYPE_BF16 || operand_dtype == FG_DTYPE_F16, FG_ERR_INVALID_ARGUMENT,
               "operand_dtype must be bf16 or fp16");
    FG_REQUIRE(scale_mode == FG_SCALE_SCALAR || scale_mode == FG_SCALE_VECTOR, FG_ERR_UNSUPPORTED,
               "16-bit expert GEMMs take per-tensor or per-row x per-column scales");
    return grouped_gemm_common(operand_dtype == FG_DTYPE_BF16 ? 2 : 3, c, a, w, a_scale, w_scale, topk_weights,
                               topk_w_dtype, topk_w_stride, sorted_ids, expert_ids, num_post_pad, max_rows, numel,
                               num_experts, N, K, ld_a, ld_c, block_rows, scale_mode, a_scale_per_row, fuse_silu, scatter,
                               mul_weight, out_dtype, nullptr, 0, nullptr, 0, 0, stream);
}

int fg_moe_grouped_gemm_int8(void* c, const void* a, const void* w, const float* a_scale, const float* w_scale,
                             const void* topk_weights, int topk_w_dtype, int64_t topk_w_stride,
                             const int32_t* sorted_ids, const int32_t* expert_ids, const int32_t* num_post_pad,
                             int64_t max_rows, int64_t numel, int num_experts, int64_t N, int64_t K, int64_t ld_a,
                             int64_t ld_c, int block_rows, int scale_mode, int a_scale_per_row, int fuse_silu,
                             int scatter, int mul_weight, int out_dtype, void* stream) {
    FG_REQUIRE(scale_mode == FG_SCALE_SCALAR || scale_mode == FG_SCALE_VECTOR, FG_ERR_UNSUPPORTED,
               "int8 expert GEMMs take per-tensor or per-token x per-channel scales");
    return grouped_gemm_common(1, c, a, w, a_scale, w_scale, topk_weights, topk_w_dtype, topk_w_stride, sorted_ids,
                               expert_ids, num_post_pad, max_rows, numel, num_experts, N, K, ld_a, ld_c, block_rows,
                               scale_mode, a_scale_per_row, fuse_silu, scatter, mul_weight, out_dtype, nullptr, 0,
                               nullptr, 0, 0, stream);
}

}  // extern "C"
