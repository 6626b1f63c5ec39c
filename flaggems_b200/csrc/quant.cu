// FP8 e4m3 activation quantisation kernels (HBM-bound; sm_100a).
//
// Three scale rules share one set of kernels:
//   QM_ACT    act_quant          s = max(amax,1e-4) * fp32(1/448), y = x * (1/s)
//   QM_GROUP  per-token-group    s = max(amax,eps) / 448,          q = x / s
//   QM_TOKEN  per-token (MoE)    s = max(max(amax,1e-10)/448, 1/(448*512)), q = x / s
//   QM_TENSOR_STATIC / _DYNAMIC  one scale for the whole tensor: given (q = x / s) or derived from a
//             precomputed global amax (s = max(amax,1e-10)/448, q = x * (1/s))
//   QM_INT8_TOKEN  per-token int8 (MoE) s = max(amax,1e-10) / 127, q = clamp(round_half_even(x / s), -128, 127)
// The results are bit-exact with IEEE fp32 evaluation of those formulas: products use
// __fmul_rn, the quotient x / s is a correctly rounded division built from one correctly
// rounded reciprocal per group and two FMAs per element (Markstein's correction), with a
// plain __fdiv_rn for the one family of divisors (all-ones significand) where that
// shortcut is not proven.
#include "common.cuh"

namespace {

enum { QM_ACT = 0, QM_GROUP = 1, QM_TOKEN = 2, QM_TENSOR_STATIC = 3, QM_TENSOR_DYNAMIC = 4, QM_INT8_TOKEN = 5 };

struct QuantArgs {
    const void* x;
    uint8_t* q;
    float* s;
    int64_t rows;  // output rows
    int64_t K;
    int group;
    int64_t ld_x, ld_q;
    int64_t s_row_stride, s_col_stride;
    float eps;
    int pow2;
    const int32_t* row_index;  // nullable gather
    int32_t index_div;
    int32_t index_limit;
    const int32_t* n_rows_dev;  // nullable
    // Optional per-row trailer of the expert-parallel dispatch format (see fg_ep_pack_rows_fp8):
    // written once per output row at byte offset meta_off of the row of q.
    const void* meta_ids;  // nullable: route slot -> global expert id
    int meta_ids_i64;
    const void* meta_w;  // route slot -> router weight
    int meta_w_dtype;
    int32_t meta_mod;  // experts per rank
    int32_t meta_rank;  // this rank (home of the rows)
    int64_t meta_off;
    int32_t* inv;  // nullable: inv[route slot] = output row
    const float* tensor_scale;  // per-tensor modes: the given scale, or the global amax
    float* tensor_scale_out;    // dynamic per-tensor mode: where the derived scale is written
    // Direct dispatch: send_counts[d] rows go to rank d; output row p (send order, destinations
    // ascending) is the (p - first[d])-th row for its destination d and is written into d's
    // receive buffer at row meta_rank * region_rows + (p - first[d]): every source rank owns a
    // fixed region of every receive buffer, so no rank needs another rank's counts to send.
    const int32_t* send_counts;  // nullable
    int world;
    int64_t region_rows;
    uint8_t* peer_q[8];
    unsigned int* status;
};

// Start of the packed row that output row `r` is written to, or nullptr when the row does not
// fit its region of the destination's receive buffer (recorded in the status word; never stored).
__device__ __forceinline__ uint8_t* packed_row_ptr(const QuantArgs& a, int64_t r) {
    if (!a.send_counts) return a.q + r * a.ld_q;
    int d = 0;
    int64_t first = 0, run = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        if (i < a.world) {
            if (r >= run) {
                d = i;
                first = run;
            }
            const int32_t c = a.send_counts[i];
            run += c > 0 ? c : 0;
        }
    }
    const int64_t idx = r - first;
    if (r >= run || idx >= a.region_rows) {
        if (a.status) atomicCAS(a.status, 0u, (2u << 16) | 1u);
        return nullptr;
    }
    return a.peer_q[d] + ((int64_t)a.meta_rank * a.region_rows + idx) * a.ld_q;
}

__device__ __forceinline__ void write_row_meta(const QuantArgs& a, int64_t out_row) {
    const int32_t slot = a.row_index[out_row];
    const long long e = a.meta_ids_i64 ? (long long)reinterpret_cast<const int64_t*>(a.meta_ids)[slot]
                                       : (long long)reinterpret_cast<const int32_t*>(a.meta_ids)[slot];
    float w;
    if (a.meta_w_dtype == FG_DTYPE_BF16) w = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.meta_w)[slot]);
    else if (a.meta_w_dtype == FG_DTYPE_F16) w = __half2float(reinterpret_cast<const __half*>(a.meta_w)[slot]);
    else w = reinterpret_cast<const float*>(a.meta_w)[slot];
    uint8_t* m = packed_row_ptr(a, out_row);
    if (!m) return;
    m += a.meta_off;
    *reinterpret_cast<int32_t*>(m) = (int32_t)(e % a.meta_mod);
    *reinterpret_cast<float*>(m + 4) = w;
    *reinterpret_cast<int32_t*>(m + 8) = slot;
    *reinterpret_cast<int32_t*>(m + 12) = a.meta_rank;
    if (a.inv) a.inv[slot] = (int32_t)out_row;
}

__device__ __forceinline__ float ceil_pow2_bits(float v) {
    // 2^ceil(log2(v)) for positive normal v: bump the exponent when any mantissa bit is set.
    uint32_t b = __float_as_uint(v);
    uint32_t e = (b >> 23) & 0xffu;
    uint32_t m = b & 0x7fffffu;
    e += (m != 0u) ? 1u : 0u;
    return __uint_as_float(e << 23);
}

template <int MODE>
__device__ __forceinline__ float make_scale(float amax, float eps, int pow2) {
    if constexpr (MODE == QM_ACT) {
        amax = fmaxf(amax, __uint_as_float(0x38d1b717u));                  // 1e-4
        float s = __fmul_rn(amax, __uint_as_float(0x3b124925u));           // fp32(1/448)
        return pow2 ? ceil_pow2_bits(s) : s;
    } else if constexpr (MODE == QM_GROUP) {
        float s = __fdiv_rn(fmaxf(amax, eps), 448.0f);
        if (pow2) s = ceil_pow2_bits(fmaxf(fabsf(s), __uint_as_float(0x2edbe6ffu)));  // floor 1e-10
        return s;
    } else if constexpr (MODE == QM_INT8_TOKEN) {
        return __fdiv_rn(fmaxf(amax, __uint_as_float(0x2edbe6ffu)), 127.0f);
    } else {
        float s = __fdiv_rn(fmaxf(amax, __uint_as_float(0x2edbe6ffu)), 448.0f);
        return fmaxf(s, __uint_as_float(0x36924925u));                      // 1/(448*512)
    }
}

// Eight quotients -> eight output bytes: e4m3 (round to nearest even, saturating), or int8 (round to
// nearest even, clamped to [-128, 127]).
template <int MODE>
__device__ __forceinline__ uint2 pack_out8(const float (&q)[8]) {
    if constexpr (MODE == QM_INT8_TOKEN) {
        uint32_t w[2] = {0u, 0u};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int v = max(-128, min(127, __float2int_rn(q[i])));
            w[i >> 2] |= (uint32_t)(v & 0xff) << (8 * (i & 3));
        }
        return make_uint2(w[0], w[1]);
    } else {
        return fg_pack_e4m3x8(q);
    }
}

// Per-group constants for turning x into x/s (or x*(1/s) for QM_ACT).
struct Divider {
    float s, r;
    bool exact_div;
};

template <int MODE>
__device__ __forceinline__ Divider make_divider(float s) {
    Divider d;
    d.s = s;
    d.r = __fdiv_rn(1.0f, s);
    d.exact_div = (MODE != QM_ACT) && ((__float_as_uint(s) & 0x7fffffu) == 0x7fffffu);
    return d;
}

template <int MODE>
__device__ __forceinline__ float apply_divider(float x, const Divider& d) {
    if constexpr (MODE == QM_ACT) {
        return __fmul_rn(x, d.r);
    } else {
        if (d.exact_div) return __fdiv_rn(x, d.s);
        float q0 = __fmul_rn(x, d.r);
        float rem = __fmaf_rn(-q0, d.s, x);
        return __fmaf_rn(rem, d.r, q0);
    }
}

// Two elements at a time with the packed fp32 instructions of sm_100 (mul/fma .f32x2): the same
// IEEE operations as apply_divider, half the issue slots.
template <int MODE>
__device__ __forceinline__ void apply_divider2(float x0, float x1, const Divider& d, float& o0, float& o1) {
    if (MODE != QM_ACT && d.exact_div) {
        o0 = __fdiv_rn(x0, d.s);
        o1 = __fdiv_rn(x1, d.s);
        return;
    }
    uint64_t x, r, q;
    asm("mov.b64 %0, {%1, %2};" : "=l"(x) : "r"(__float_as_uint(x0)), "r"(__float_as_uint(x1)));
    asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "r"(__float_as_uint(d.r)));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(q) : "l"(x), "l"(r));
    if constexpr (MODE != QM_ACT) {
        uint64_t ns, rem;
        asm("mov.b64 %0, {%1, %1};" : "=l"(ns) : "r"(__float_as_uint(-d.s)));
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rem) : "l"(q), "l"(ns), "l"(x));   // x - q*s, exact
        asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(q) : "l"(rem), "l"(r), "l"(q));
    }
    uint32_t lo, hi;
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(q));
    o0 = __uint_as_float(lo);
    o1 = __uint_as_float(hi);
}

__device__ __forceinline__ int64_t resolve_rows(const QuantArgs& a) {
    int64_t rows = a.rows;
    if (a.n_rows_dev) {
        int64_t v = *a.n_rows_dev;
        rows = v < rows ? v : rows;
    }
    return rows;
}

// Source row of output row r, or -1 for an all-zero (padding) row.
__device__ __forceinline__ int64_t source_row(const QuantArgs& a, int64_t r) {
    if (!a.row_index) return r;
    int32_t idx = a.row_index[r];
    return (idx >= 0 && idx < a.index_limit) ? (int64_t)(idx / a.index_div) : -1;
}

// ---- small groups: a team of TPG lanes owns one group of TPG*8*VPT elements -------------
// Groups are numbered row-major (row * groups_per_row + column group).  A team walks them with
// a constant stride and keeps (row, column group) incrementally: no division in the loop.
template <typename T, int MODE, int TPG, int VPT>
__global__ void __launch_bounds__(256) group_quant_kernel(QuantArgs a) {
    constexpr int UNROLL = 2;
    constexpr int GROUP = TPG * 8 * VPT;
    const int64_t rows = resolve_rows(a);
    const int gpr = (int)(a.K / GROUP);
    const int64_t total = rows * gpr;
    const int lane_in_team = threadIdx.x % TPG;
    const int64_t team = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / TPG;
    const int64_t teams = (int64_t)gridDim.x * blockDim.x / TPG;
    const int64_t stride = teams * UNROLL;
    const T* x = reinterpret_cast<const T*>(a.x);
    // Trip count from the first team of the warp, so the whole warp runs the same iterations.
    const int64_t warp_first = team - (threadIdx.x % 32) / TPG;
    const int64_t iters = warp_first < total ? (total - warp_first + stride - 1) / stride : 0;
    const int step_row = (int)(stride / gpr), step_cg = (int)(stride % gpr);
    int row[UNROLL], cg[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t g0 = team + (int64_t)u * teams;
        row[u] = (int)(g0 / gpr);
        cg[u] = (int)(g0 % gpr);
    }
    for (int64_t it = 0; it < iters; ++it) {
        float v[UNROLL][VPT][8];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t src = row[u] < rows ? source_row(a, row[u]) : -1;
#pragma unroll
            for (int w = 0; w < VPT; ++w) {
                if (src >= 0) {
                    fg_load8(x + src * a.ld_x + cg[u] * GROUP + (w * TPG + lane_in_team) * 8, v[u][w]);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) v[u][w][i] = 0.0f;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            float amax = 0.0f;
#pragma unroll
            for (int w = 0; w < VPT; ++w)
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[u][w][i]));
#pragma unroll
            for (int o = TPG / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float s = make_scale<MODE>(amax, a.eps, a.pow2);
            const Divider d = make_divider<MODE>(s);
            uint8_t* qrow = nullptr;
            if (row[u] < rows) qrow = a.meta_ids ? packed_row_ptr(a, row[u]) : a.q + (int64_t)row[u] * a.ld_q;
            if (qrow) {
#pragma unroll
                for (int w = 0; w < VPT; ++w) {
                    float q[8];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) apply_divider2<MODE>(v[u][w][i], v[u][w][i + 1], d, q[i], q[i + 1]);
                    *reinterpret_cast<uint2*>(qrow + cg[u] * GROUP + (w * TPG + lane_in_team) * 8) = fg_pack_e4m3x8(q);
                }
                if (lane_in_team == 0) {
                    if (a.meta_ids) {  // packed row: scales sit behind the payload of the same row
                        reinterpret_cast<float*>(qrow + a.K)[cg[u]] = s;
                        if (cg[u] == 0) write_row_meta(a, row[u]);
                    } else {
                        a.s[(int64_t)row[u] * a.s_row_stride + (int64_t)cg[u] * a.s_col_stride] = s;
                    }
                }
            }
            cg[u] += step_cg;
            row[u] += step_row;
            if (cg[u] >= gpr) {
                cg[u] -= gpr;
                row[u] += 1;
            }
        }
    }
}

// ---- small groups, 16-bit inputs: the bandwidth path ---------------------------------------
// A lane owns 16 consecutive elements (two 16-byte loads, one 16-byte store), a team of
// GROUP/16 lanes owns a group.  The inputs stay in registers as raw 16-bit pairs: max|x| is taken
// on the pairs (exact in the input type), and they are widened to fp32 only where they are
// scaled, so that a thread carries 8 registers of data per group in flight instead of 16 and five
// CTAs (40 warps, 48 registers each) fit an SM; six CTAs spill and measured no faster.  PACKED selects the expert-parallel dispatch format (scales and a trailer behind
// the payload of each row, rows optionally stored into peers' receive buffers).
template <typename T> struct Pair16;
template <> struct Pair16<__nv_bfloat16> {
    using V = __nv_bfloat162;
    static __device__ __forceinline__ V absmax(V m, uint32_t w) {
        return __hmax2(m, __habs2(*reinterpret_cast<const V*>(&w)));
    }
    static __device__ __forceinline__ float reduce(V m) { return fmaxf(__bfloat162float(m.x), __bfloat162float(m.y)); }
    static __device__ __forceinline__ void widen(uint32_t w, float& lo, float& hi) {
        lo = __uint_as_float(w << 16);
        hi = __uint_as_float(w & 0xffff0000u);
    }
};
template <> struct Pair16<__half> {
    using V = __half2;
    static __device__ __forceinline__ V absmax(V m, uint32_t w) {
        return __hmax2(m, __habs2(*reinterpret_cast<const V*>(&w)));
    }
    static __device__ __forceinline__ float reduce(V m) { return fmaxf(__half2float(m.x), __half2float(m.y)); }
    static __device__ __forceinline__ void widen(uint32_t w, float& lo, float& hi) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
        lo = f.x;
        hi = f.y;
    }
};

template <typename T, int MODE, int TPG, bool PACKED>
__global__ void __launch_bounds__(256, 5) group_quant16_kernel(QuantArgs a) {
    constexpr int UNROLL = 2;
    constexpr int GROUP = TPG * 16;
    using P = Pair16<T>;
    const int64_t rows = resolve_rows(a);
    const int gpr = (int)(a.K / GROUP);
    const int64_t total = rows * gpr;
    const int lane_in_team = threadIdx.x % TPG;
    const int64_t team = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / TPG;
    const int64_t teams = (int64_t)gridDim.x * blockDim.x / TPG;
    const int64_t stride = teams * UNROLL;
    const T* x = reinterpret_cast<const T*>(a.x);
    // Trip count from the first team of the warp, so the whole warp runs the same iterations.
    const int64_t warp_first = team - (threadIdx.x % 32) / TPG;
    const int64_t iters = warp_first < total ? (total - warp_first + stride - 1) / stride : 0;
    const int step_row = (int)(stride / gpr), step_cg = (int)(stride % gpr);
    int row[UNROLL], cg[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
        const int64_t g0 = team + (int64_t)u * teams;
        row[u] = (int)(g0 / gpr);
        cg[u] = (int)(g0 % gpr);
    }
    for (int64_t it = 0; it < iters; ++it) {
        uint4 v[UNROLL][2];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const int64_t src = row[u] < rows ? source_row(a, row[u]) : -1;
            if (src >= 0) {
                const uint4* p = reinterpret_cast<const uint4*>(x + src * a.ld_x + cg[u] * GROUP + lane_in_team * 16);
                v[u][0] = p[0];
                v[u][1] = p[1];
            } else {
                v[u][0] = v[u][1] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
            const uint32_t w[8] = {v[u][0].x, v[u][0].y, v[u][0].z, v[u][0].w, v[u][1].x, v[u][1].y, v[u][1].z, v[u][1].w};
            typename P::V m2 = P::absmax(P::absmax(typename P::V(), w[0]), w[1]);
#pragma unroll
            for (int i = 2; i < 8; ++i) m2 = P::absmax(m2, w[i]);
            float amax = P::reduce(m2);
#pragma unroll
            for (int o = TPG / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            const float s = make_scale<MODE>(amax, a.eps, a.pow2);
            const Divider d = make_divider<MODE>(s);
            uint8_t* qrow = nullptr;
            if (row[u] < rows) qrow = PACKED ? packed_row_ptr(a, row[u]) : a.q + (int64_t)row[u] * a.ld_q;
            if (qrow) {
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float a0, a1, b0, b1, q0, q1, q2, q3;
                    P::widen(w[2 * i], a0, a1);
                    P::widen(w[2 * i + 1], b0, b1);
                    apply_divider2<MODE>(a0, a1, d, q0, q1);
                    apply_divider2<MODE>(b0, b1, d, q2, q3);
                    const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
                    const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
                    o[i] = lo | (hi << 16);
                }
                *reinterpret_cast<uint4*>(qrow + cg[u] * GROUP + lane_in_team * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                if (lane_in_team == 0) {
                    if constexpr (PACKED) {  // scales sit behind the payload of the same row
                        reinterpret_cast<float*>(qrow + a.K)[cg[u]] = s;
                        if (cg[u] == 0) write_row_meta(a, row[u]);
                    } else {
                        a.s[(int64_t)row[u] * a.s_row_stride + (int64_t)cg[u] * a.s_col_stride] = s;
                    }
                }
            }
            cg[u] += step_cg;
            row[u] += step_row;
            if (cg[u] >= gpr) {
                cg[u] -= gpr;
                row[u] += 1;
            }
        }
    }
}

// Expert-parallel dispatch, second step: every token was quantised once into a staging row (FP8
// payload, then its scales); this kernel copies the staged row of route slot order[r] to output row
// r (a local packed buffer, or this rank's region of the destination rank's receive buffer) and
// writes the row's trailer.  One warp per row, four 16-byte loads in flight per lane.
__global__ void __launch_bounds__(256) pack_copy_kernel(QuantArgs a, const uint8_t* __restrict__ staged) {
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int nvec = (int)(a.K / 16);
    const int s_cols = (int)(a.K / a.group);
    for (int64_t r = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5); r < a.rows; r += (int64_t)gridDim.x * warps) {
        const int64_t src = source_row(a, r);
        uint8_t* dst = packed_row_ptr(a, r);
        if (src < 0 || !dst) continue;
        const uint8_t* srow = staged + src * a.ld_q;
        const uint4* sq = reinterpret_cast<const uint4*>(srow);
        uint4* dq = reinterpret_cast<uint4*>(dst);
        for (int v0 = lane; v0 < nvec; v0 += 128) {
            uint4 t[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + 32 * u;
                t[u] = v < nvec ? sq[v] : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int v = v0 + 32 * u;
                if (v < nvec) dq[v] = t[u];
            }
        }
        const float* ss = reinterpret_cast<const float*>(srow + a.K);
        float* ds = reinterpret_cast<float*>(dst + a.K);
        for (int v = lane; v < s_cols; v += 32) ds[v] = ss[v];
        if (lane == 0) write_row_meta(a, r);
    }
}

// ---- any group size (multiple of 8), one CTA per group: per-token rows, block_size = K ...
template <typename T, int MODE>
__global__ void __launch_bounds__(256) row_quant_kernel(QuantArgs a) {
    constexpr int MAXV = 8;  // vectors of 8 cached in registers per thread
    const int64_t rows = resolve_rows(a);
    const int64_t gpr = a.K / a.group;
    const int64_t g = blockIdx.x;
    const int64_t row = g / gpr, cg = g % gpr;
    if (row >= rows) return;
    const int64_t src = source_row(a, row);
    const T* x = reinterpret_cast<const T*>(a.x) + (src >= 0 ? src : 0) * a.ld_x + cg * a.group;
    uint8_t* q = a.q + row * a.ld_q + cg * a.group;
    const int nvec = a.group / 8;
    const bool cached = nvec <= MAXV * 256;

    float v[MAXV][8];
    float amax = 0.0f;
    if (src >= 0) {
        if (cached) {
#pragma unroll
            for (int j = 0; j < MAXV; ++j) {
                const int iv = threadIdx.x + j * 256;
                if (iv < nvec) {
                    fg_load8(x + (int64_t)iv * 8, v[j]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
                }
            }
        } else {
            for (int iv = threadIdx.x; iv < nvec; iv += 256) {
                float t[8];
                fg_load8(x + (int64_t)iv * 8, t);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(t[i]));
            }
        }
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) amax = fmaxf(amax, red[w]);

    float s;
    if constexpr (MODE == QM_TENSOR_STATIC) {
        s = a.tensor_scale[0];
    } else if constexpr (MODE == QM_TENSOR_DYNAMIC) {
        s = __fdiv_rn(fmaxf(a.tensor_scale[0], __uint_as_float(0x2edbe6ffu)), 448.0f);
        if (threadIdx.x == 0 && g == 0) a.tensor_scale_out[0] = s;
    } else {
        s = make_scale<MODE>(amax, a.eps, a.pow2);
        if (threadIdx.x == 0) a.s[row * a.s_row_stride + cg * a.s_col_stride] = s;
    }
    // dynamic per-tensor quantisation multiplies by the reciprocal, like act_quant
    constexpr int DMODE = MODE == QM_TENSOR_DYNAMIC ? QM_ACT : (MODE == QM_TENSOR_STATIC ? QM_GROUP : MODE);
    const Divider d = make_divider<DMODE>(s);

    if (src < 0) {
        for (int iv = threadIdx.x; iv < nvec; iv += 256) *reinterpret_cast<uint2*>(q + (int64_t)iv * 8) = make_uint2(0u, 0u);
        return;
    }
    if (cached) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
            const int iv = threadIdx.x + j * 256;
            if (iv < nvec) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; i += 2) apply_divider2<DMODE>(v[j][i], v[j][i + 1], d, o[i], o[i + 1]);
                *reinterpret_cast<uint2*>(q + (int64_t)iv * 8) = pack_out8<MODE>(o);
            }
        }
    } else {
        for (int iv = threadIdx.x; iv < nvec; iv += 256) {
            float t[8], o[8];
            fg_load8(x + (int64_t)iv * 8, t);
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = apply_divider<DMODE>(t[i], d);
            *reinterpret_cast<uint2*>(q + (int64_t)iv * 8) = pack_out8<MODE>(o);
        }
    }
}

// Global max|x| over rows [0, rows) into amax[0] (which must start at zero): block reduction, then
// one atomicMax per block on the bit pattern (non-negative floats order like unsigned integers).
template <typename T>
__global__ void __launch_bounds__(256) abs_max_kernel(const T* __restrict__ x, int64_t rows, int64_t K, int64_t ld_x,
                                                      const int32_t* __restrict__ n_rows_dev,
                                                      unsigned int* __restrict__ amax) {
    if (n_rows_dev) {
        const int64_t v = *n_rows_dev;
        rows = v < rows ? v : rows;
    }
    const int64_t vec_per_row = K / 8, total = rows * vec_per_row;
    float m = 0.0f;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < total; v += (int64_t)gridDim.x * blockDim.x) {
        float f[8];
        fg_load8(x + (v / vec_per_row) * ld_x + (v % vec_per_row) * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(f[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __shared__ float red[8];
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
        atomicMax(amax, __float_as_uint(m));
    }
}

template <typename T, int MODE>
int launch_quant_t(const QuantArgs& a, cudaStream_t st) {
    if (a.rows == 0 || a.K == 0) return FG_OK;
    const int64_t groups = a.rows * (a.K / a.group);
    auto small = [&](auto kernel, int tpg) -> int {
        const int64_t threads = groups * tpg;
        int64_t blocks = fg_cdiv(threads, 256 * 2);
        const int64_t cap = (int64_t)fg_num_sms() * 24;
        if (blocks > cap) blocks = cap;
        if (blocks < 1) blocks = 1;
        kernel<<<(unsigned)blocks, 256, 0, st>>>(a);
        fg_count_launch(1);
        FG_LAUNCH_CHECK();
        return FG_OK;
    };
    if constexpr (sizeof(T) == 2) {
        // 16-byte stores need 16-byte aligned output rows; otherwise the generic kernel below
        const bool q16 = ((uintptr_t)a.q % 16 == 0) && (a.ld_q % 16 == 0);
        if (q16 && a.meta_ids) {
            if (a.group == 128) return small(group_quant16_kernel<T, MODE, 8, true>, 8);
        } else if (q16) {
            switch (a.group) {
                case 64: return small(group_quant16_kernel<T, MODE, 4, false>, 4);
                case 128: return small(group_quant16_kernel<T, MODE, 8, false>, 8);
                case 256: return small(group_quant16_kernel<T, MODE, 16, false>, 16);
                case 512: return small(group_quant16_kernel<T, MODE, 32, false>, 32);
                default: break;
            }
        }
    }
    switch (a.group) {
        // sixteen elements (two 16-byte loads) per lane: the shuffle reduction, the scale and the
        // index arithmetic are paid once per 16 elements, and four loads per lane are in flight
        case 64: return small(group_quant_kernel<T, MODE, 4, 2>, 4);
        case 128: return small(group_quant_kernel<T, MODE, 8, 2>, 8);
        case 256: return small(group_quant_kernel<T, MODE, 16, 2>, 16);
        case 512: return small(group_quant_kernel<T, MODE, 32, 2>, 32);
        default: break;
    }
    FG_REQUIRE(groups < (1ll << 31), FG_ERR_UNSUPPORTED, "too many groups (%lld) for one launch", (long long)groups);
    row_quant_kernel<T, MODE><<<(unsigned)groups, 256, 0, st>>>(a);
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

template <int MODE>
int launch_quant(int dtype, const QuantArgs& a, cudaStream_t st) {
    switch (dtype) {
        case FG_DTYPE_BF16: return launch_quant_t<__nv_bfloat16, MODE>(a, st);
        case FG_DTYPE_F16: return launch_quant_t<__half, MODE>(a, st);
        case FG_DTYPE_F32: return launch_quant_t<float, MODE>(a, st);
        default: fg_set_error("unsupported input dtype code %d", dtype); return FG_ERR_INVALID_ARGUMENT;
    }
}

int check_common(const QuantArgs& a, int dtype) {
    FG_REQUIRE(a.rows >= 0 && a.K >= 0, FG_ERR_INVALID_ARGUMENT, "negative size");
    FG_REQUIRE(a.group > 0 && a.group % 8 == 0, FG_ERR_UNSUPPORTED, "group size %d must be a positive multiple of 8", a.group);
    FG_REQUIRE(a.K % a.group == 0, FG_ERR_INVALID_ARGUMENT, "last dimension %lld must be divisible by the group size %d",
               (long long)a.K, a.group);
    if (a.rows == 0 || a.K == 0) return FG_OK;
    FG_REQUIRE(a.x && a.q && a.s, FG_ERR_INVALID_ARGUMENT, "null pointer");
    const int esz = dtype == FG_DTYPE_F32 ? 4 : 2;
    FG_REQUIRE(((uintptr_t)a.x % 16 == 0) && ((a.ld_x * esz) % 16 == 0), FG_ERR_UNSUPPORTED,
               "input rows must be 16-byte aligned (ptr %p, row stride %lld elements)", a.x, (long long)a.ld_x);
    FG_REQUIRE(((uintptr_t)a.q % 8 == 0) && (a.ld_q % 8 == 0), FG_ERR_UNSUPPORTED,
               "output rows must be 8-byte aligned (ptr %p, row stride %lld)", (void*)a.q, (long long)a.ld_q);
    return FG_OK;
}

}  // namespace

extern "C" {

int fg_act_quant_bf16_e4m3(const void* x, void* y, float* s, int64_t M, int64_t N, int block, int64_t ld_x,
                           int64_t ld_y, int64_t ld_s, int round_pow2, void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)y; a.s = s; a.rows = M; a.K = N; a.group = block;
    a.ld_x = ld_x; a.ld_q = ld_y; a.s_row_stride = ld_s; a.s_col_stride = 1;
    a.eps = 0.0f; a.pow2 = round_pow2 != 0;
    int rc = check_common(a, FG_DTYPE_BF16);
    if (rc != FG_OK) return rc;
    return launch_quant<QM_ACT>(FG_DTYPE_BF16, a, (cudaStream_t)stream);
}

int fg_per_token_group_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K, int group,
                                 int64_t ld_x, int64_t ld_q, int64_t s_row_stride, int64_t s_col_stride, float eps,
                                 int ue8m0, void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)q; a.s = s; a.rows = M; a.K = K; a.group = group;
    a.ld_x = ld_x; a.ld_q = ld_q; a.s_row_stride = s_row_stride; a.s_col_stride = s_col_stride;
    a.eps = eps; a.pow2 = ue8m0 != 0;
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    return launch_quant<QM_GROUP>(x_dtype, a, (cudaStream_t)stream);
}

int fg_per_token_group_quant_fp8_gather(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K,
                                        int group, int64_t ld_x, int64_t ld_q, const int32_t* row_index,
                                        int32_t index_div, int32_t index_limit, const int32_t* n_rows_dev,
                                        void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)q; a.s = s; a.rows = M; a.K = K; a.group = group;
    a.ld_x = ld_x; a.ld_q = ld_q; a.s_row_stride = group > 0 ? K / group : 0; a.s_col_stride = 1;
    a.eps = 1e-10f; a.pow2 = 0;
    a.row_index = row_index; a.index_div = index_div; a.index_limit = index_limit; a.n_rows_dev = n_rows_dev;
    FG_REQUIRE(row_index == nullptr || index_div > 0, FG_ERR_INVALID_ARGUMENT, "index_div must be positive");
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    return launch_quant<QM_GROUP>(x_dtype, a, (cudaStream_t)stream);
}

int fg_ep_pack_rows_fp8(const void* x, int x_dtype, int64_t T, int64_t K, int64_t ld_x, const void* topk_ids,
                        int ids_are_i64, const void* topk_w, int topk_w_dtype, int topk, int experts_per_rank,
                        int home_rank, const int32_t* order, void* packed, int64_t row_bytes, int32_t* inv,
                        void* stream) {
    return fg_ep_pack_rows_fp8_peer(x, x_dtype, T, K, ld_x, topk_ids, ids_are_i64, topk_w, topk_w_dtype, topk,
                                    experts_per_rank, home_rank, order, packed, row_bytes, inv, nullptr, nullptr, 0, 0,
                                    stream);
}

int fg_ep_pack_rows_fp8_peer(const void* x, int x_dtype, int64_t T, int64_t K, int64_t ld_x, const void* topk_ids,
                             int ids_are_i64, const void* topk_w, int topk_w_dtype, int topk, int experts_per_rank,
                             int home_rank, const int32_t* order, void* packed, int64_t row_bytes, int32_t* inv,
                             const int32_t* send_counts, void* const* peer_rows, int world, int64_t region_rows,
                             void* stream) {
    FG_REQUIRE(T >= 0 && K > 0 && topk > 0 && experts_per_rank > 0, FG_ERR_INVALID_ARGUMENT, "bad sizes");
    FG_REQUIRE(K % 128 == 0, FG_ERR_UNSUPPORTED, "row length %lld must be a multiple of 128", (long long)K);
    FG_REQUIRE(row_bytes >= K + 4 * (K / 128) + 16 && row_bytes % 16 == 0, FG_ERR_INVALID_ARGUMENT,
               "row_bytes %lld too small or not a multiple of 16", (long long)row_bytes);
    FG_REQUIRE(T * topk < (1ll << 31), FG_ERR_UNSUPPORTED, "too many route slots");
    if (T == 0) return FG_OK;
    FG_REQUIRE(x && topk_ids && topk_w && order && (packed || send_counts), FG_ERR_INVALID_ARGUMENT, "null pointer");
    FG_REQUIRE(send_counts == nullptr ||
                   (peer_rows && world >= 1 && world <= 8 && home_rank >= 0 && home_rank < world && region_rows > 0),
               FG_ERR_INVALID_ARGUMENT, "direct dispatch needs 1..8 peer buffers, a rank below world and region_rows > 0");
    FG_REQUIRE(send_counts == nullptr || T * topk <= region_rows, FG_ERR_INVALID_ARGUMENT,
               "%lld route slots do not fit a region of %lld rows", (long long)(T * topk), (long long)region_rows);
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)packed; a.s = reinterpret_cast<float*>((uint8_t*)packed + K);
    a.rows = T * topk; a.K = K; a.group = 128;
    a.ld_x = ld_x; a.ld_q = row_bytes; a.s_row_stride = row_bytes / 4; a.s_col_stride = 1;
    a.eps = 1e-10f; a.pow2 = 0;
    a.row_index = order; a.index_div = topk; a.index_limit = (int32_t)(T * topk); a.n_rows_dev = nullptr;
    a.meta_ids = topk_ids; a.meta_ids_i64 = ids_are_i64; a.meta_w = topk_w; a.meta_w_dtype = topk_w_dtype;
    a.meta_mod = experts_per_rank; a.meta_rank = home_rank; a.meta_off = K + 4 * (K / 128); a.inv = inv;
    a.send_counts = send_counts; a.world = world; a.region_rows = region_rows;
    a.status = fg_status_word_device_ptr();
    for (int i = 0; i < 8; ++i) a.peer_q[i] = (send_counts && i < world) ? (uint8_t*)peer_rows[i] : nullptr;
    if (send_counts) {
        a.q = (uint8_t*)peer_rows[home_rank];
        a.s = reinterpret_cast<float*>(a.q + K);
    }
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    if (send_counts && packed && topk > 1) {
        // `packed` as a staging area of T rows: every token is quantised once (not once per route slot)
        // and its staged row is copied to each of its destinations.
        FG_REQUIRE((uintptr_t)packed % 16 == 0, FG_ERR_UNSUPPORTED, "the staging rows must be 16-byte aligned");
        QuantArgs b{};
        b.x = x; b.q = (uint8_t*)packed; b.s = reinterpret_cast<float*>((uint8_t*)packed + K);
        b.rows = T; b.K = K; b.group = 128; b.ld_x = ld_x; b.ld_q = row_bytes;
        b.s_row_stride = row_bytes / 4; b.s_col_stride = 1; b.eps = 1e-10f; b.pow2 = 0;
        rc = check_common(b, x_dtype);
        if (rc != FG_OK) return rc;
        rc = launch_quant<QM_GROUP>(x_dtype, b, (cudaStream_t)stream);
        if (rc != FG_OK) return rc;
        int64_t blocks = fg_cdiv(a.rows, 8);
        const int64_t cap = (int64_t)fg_num_sms() * 8;
        if (blocks > cap) blocks = cap;
        pack_copy_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(a, (const uint8_t*)packed);
        fg_count_launch(1);
        FG_LAUNCH_CHECK();
        return FG_OK;
    }
    return launch_quant<QM_GROUP>(x_dtype, a, (cudaStream_t)stream);
}

int fg_abs_max(const void* x, int x_dtype, int64_t M, int64_t K, int64_t ld_x, const int32_t* n_rows_dev,
               float* amax, void* stream) {
    FG_REQUIRE(M >= 0 && K >= 0 && amax, FG_ERR_INVALID_ARGUMENT, "bad arguments");
    if (M == 0 || K == 0) return FG_OK;
    const int esz = x_dtype == FG_DTYPE_F32 ? 4 : 2;
    FG_REQUIRE(K % 8 == 0 && (uintptr_t)x % 16 == 0 && (ld_x * esz) % 16 == 0, FG_ERR_UNSUPPORTED,
               "abs_max needs K %% 8 == 0 and 16-byte aligned rows");
    int64_t blocks = fg_cdiv(M * (K / 8), 256 * 4);
    const int64_t cap = (int64_t)fg_num_sms() * 8;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = (cudaStream_t)stream;
    unsigned int* out = reinterpret_cast<unsigned int*>(amax);
    switch (x_dtype) {
        case FG_DTYPE_BF16: abs_max_kernel<<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)x, M, K, ld_x, n_rows_dev, out); break;
        case FG_DTYPE_F16: abs_max_kernel<<<(unsigned)blocks, 256, 0, st>>>((const __half*)x, M, K, ld_x, n_rows_dev, out); break;
        case FG_DTYPE_F32: abs_max_kernel<<<(unsigned)blocks, 256, 0, st>>>((const float*)x, M, K, ld_x, n_rows_dev, out); break;
        default: fg_set_error("unsupported input dtype code %d", x_dtype); return FG_ERR_INVALID_ARGUMENT;
    }
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_per_tensor_quant_fp8(const void* x, int x_dtype, void* q, const float* scale_or_amax, int dynamic,
                            float* scale_out, int64_t M, int64_t K, int64_t ld_x, int64_t ld_q,
                            const int32_t* row_index, int32_t index_div, int32_t index_limit,
                            const int32_t* n_rows_dev, void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)q; a.s = const_cast<float*>(scale_or_amax); a.rows = M; a.K = K; a.group = (int)K;
    a.ld_x = ld_x; a.ld_q = ld_q; a.s_row_stride = 0; a.s_col_stride = 0;
    a.row_index = row_index; a.index_div = index_div; a.index_limit = index_limit; a.n_rows_dev = n_rows_dev;
    a.tensor_scale = scale_or_amax; a.tensor_scale_out = scale_out;
    FG_REQUIRE(scale_or_amax && (!dynamic || scale_out), FG_ERR_INVALID_ARGUMENT, "scale pointers missing");
    FG_REQUIRE(K < (1ll << 31) && M < (1ll << 31), FG_ERR_UNSUPPORTED, "size too large");
    FG_REQUIRE(row_index == nullptr || index_div > 0, FG_ERR_INVALID_ARGUMENT, "index_div must be positive");
    if (K == 0 || M == 0) return FG_OK;
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
#define FG_ROW_LAUNCH(T_)                                                                       \
    if (dynamic) row_quant_kernel<T_, QM_TENSOR_DYNAMIC><<<(unsigned)M, 256, 0, st>>>(a);        \
    else row_quant_kernel<T_, QM_TENSOR_STATIC><<<(unsigned)M, 256, 0, st>>>(a);
    switch (x_dtype) {
        case FG_DTYPE_BF16: FG_ROW_LAUNCH(__nv_bfloat16) break;
        case FG_DTYPE_F16: FG_ROW_LAUNCH(__half) break;
        case FG_DTYPE_F32: FG_ROW_LAUNCH(float) break;
        default: fg_set_error("unsupported input dtype code %d", x_dtype); return FG_ERR_INVALID_ARGUMENT;
    }
#undef FG_ROW_LAUNCH
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_per_token_quant_int8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K, int64_t ld_x,
                            int64_t ld_q, const int32_t* row_index, int32_t index_div, int32_t index_limit,
                            const int32_t* n_rows_dev, void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)q; a.s = s; a.rows = M; a.K = K; a.group = (int)K;
    a.ld_x = ld_x; a.ld_q = ld_q; a.s_row_stride = 1; a.s_col_stride = 1;
    a.eps = 1e-10f; a.pow2 = 0;
    a.row_index = row_index; a.index_div = index_div; a.index_limit = index_limit; a.n_rows_dev = n_rows_dev;
    FG_REQUIRE(K < (1ll << 31) && M < (1ll << 31), FG_ERR_UNSUPPORTED, "size too large");
    FG_REQUIRE(row_index == nullptr || index_div > 0, FG_ERR_INVALID_ARGUMENT, "index_div must be positive");
    if (K == 0 || M == 0) return FG_OK;
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    switch (x_dtype) {
        case FG_DTYPE_BF16: row_quant_kernel<__nv_bfloat16, QM_INT8_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        case FG_DTYPE_F16: row_quant_kernel<__half, QM_INT8_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        case FG_DTYPE_F32: row_quant_kernel<float, QM_INT8_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        default: fg_set_error("unsupported input dtype code %d", x_dtype); return FG_ERR_INVALID_ARGUMENT;
    }
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

int fg_per_token_quant_fp8(const void* x, int x_dtype, void* q, float* s, int64_t M, int64_t K, int64_t ld_x,
                           int64_t ld_q, const int32_t* row_index, int32_t index_div, int32_t index_limit,
                           const int32_t* n_rows_dev, void* stream) {
    QuantArgs a{};
    a.x = x; a.q = (uint8_t*)q; a.s = s; a.rows = M; a.K = K; a.group = (int)K;
    a.ld_x = ld_x; a.ld_q = ld_q; a.s_row_stride = 1; a.s_col_stride = 1;
    a.eps = 1e-10f; a.pow2 = 0;
    a.row_index = row_index; a.index_div = index_div; a.index_limit = index_limit; a.n_rows_dev = n_rows_dev;
    FG_REQUIRE(K < (1ll << 31), FG_ERR_UNSUPPORTED, "row length %lld too large", (long long)K);
    FG_REQUIRE(row_index == nullptr || index_div > 0, FG_ERR_INVALID_ARGUMENT, "index_div must be positive");
    if (K == 0) return FG_OK;
    int rc = check_common(a, x_dtype);
    if (rc != FG_OK) return rc;
    // Row-sized groups always take the one-CTA-per-row kernel.
    cudaStream_t st = (cudaStream_t)stream;
    if (M == 0) return FG_OK;
    FG_REQUIRE(M < (1ll << 31), FG_ERR_UNSUPPORTED, "too many rows");
    switch (x_dtype) {
        case FG_DTYPE_BF16: row_quant_kernel<__nv_bfloat16, QM_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        case FG_DTYPE_F16: row_quant_kernel<__half, QM_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        case FG_DTYPE_F32: row_quant_kernel<float, QM_TOKEN><<<(unsigned)M, 256, 0, st>>>(a); break;
        default: fg_set_error("unsupported input dtype code %d", x_dtype); return FG_ERR_INVALID_ARGUMENT;
    }
    fg_count_launch(1);
    FG_LAUNCH_CHECK();
    return FG_OK;
}

}  // extern "C"
