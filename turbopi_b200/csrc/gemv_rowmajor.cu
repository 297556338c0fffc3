// Decode-shaped (M <= 16) 4-bit weight-only GEMV for row-major packed weights
// ([N, K/2] bytes): NVFP4 (e2m1 + block scales) and unsigned INT4 (zero point 8 +
// group scales).
//
// HBM-bound design for B200:
//   * persistent CTAs walk a list of row tiles; a tile (R consecutive rows = one
//     contiguous byte range of the weight matrix, plus its scale rows) is fetched
//     by ONE thread with 1-D bulk async copies into a 4-stage shared-memory ring
//     and signalled through an mbarrier, so the bytes in flight per SM do not
//     depend on registers or occupancy;
//   * the first tiles are requested BEFORE griddepcontrol.wait, so under
//     programmatic dependent launch the weight stream of kernel i+1 overlaps the
//     tail of kernel i (weights never depend on the previous kernel);
//   * activations live in registers as fp16 pairs; each lane owns fixed 32-wide K
//     slices, reads its 16 bytes of codes per row with one conflict-free LDS.128,
//     decodes in registers (cvt.rn.f16x2.e2m1x2 / magic-number int4), multiplies
//     in packed fp16 over 4 products, then accumulates in fp32 with the block
//     scale; rows are reduced with warp shuffles, K-parts (split K across warps
//     for long rows) through shared memory in a fixed order (deterministic).
#include <algorithm>
#include <atomic>

#include "common.cuh"

namespace tpb {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int kStages = 4;
constexpr int kWStage = 16384;     // weight bytes per stage
constexpr int kSStage = 4096;      // scale bytes per stage
constexpr int kMaxTileRows = 64;
constexpr int kMaxPartials = 256;  // rows * K-parts per tile

enum { kFmtE2M1 = 0, kFmtU4 = 1 };
// how the scales of one 32-code chunk are found
enum {
    kScE4M3B16 = 0,  // two E4M3 bytes per chunk
    kScE4M3B32 = 1,  // one E4M3 byte per chunk
    kScF32B16 = 2,   // two floats per chunk
    kScF32B32 = 3,   // one float per chunk
    kScF16Group = 4, // fp16, one per `group` codes (group % 32 == 0)
    kScBF16Group = 5 // bf16, same
};

struct ProblemDev {
    const uint8_t* w;
    const uint8_t* scales;
    const void* x;
    const void* x_scales;
    const void* bias;
    void* out;
    int N;
    int K;
    int ldo;             // output row stride in elements
    float global_scale;
    int tile_begin;      // index of this problem's first tile in the launch-wide list
    int rows_per_tile;   // multiple of (8 / kparts)
    int kparts;          // warps along K: 1, 2, 4 or 8
    int scale_row_bytes;
    int scales_by_tma;   // 1: scale rows ride in the stage buffer, 0: read from global
};

template <int MAXP>
struct GemvParams {
    int num_problems;
    int total_tiles;
    int M;
    int x_dtype;
    int bias_dtype;
    int out_dtype;
    int activation;
    int group;  // codes per scale
    uint32_t u4_xor;  // 0x88888888 turns two's-complement int4 nibbles into the offset-8 codes the decoder expects
    ProblemDev prob[MAXP];
};

// Index of the problem that owns `tile`, by bisection: the table lives in the kernel's parameter space, where
// every dependent look-up with a computed index costs ~100 cycles, so a walk from entry 0 delays the CTAs of
// the last problems by microseconds.
template <int MAXP>
__device__ __forceinline__ int find_problem(const GemvParams<MAXP>& P, int tile) {
    int lo = 0, hi = P.num_problems - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tile >= P.prob[mid].tile_begin) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ __half to_half_sat(float v) {
    return __float2half_rn(fminf(fmaxf(v, -65504.0f), 65504.0f));
}

// Load the 32 activations of chunk j of row m into fp16 pairs ordered the way the
// decoder of FMT produces weight pairs.
template <int FMT>
__device__ __forceinline__ void load_x_chunk(__half2 (&xr)[16], const void* x, const void* xs, int x_dtype,
                                             size_t row_off, int j, int group, bool valid, float prescale) {
    float v[32];
    if (!valid) {
#pragma unroll
        for (int i = 0; i < 16; ++i) xr[i] = __float2half2_rn(0.0f);
        return;
    }
    const size_t e0 = row_off + static_cast<size_t>(j) * 32;
    if (x_dtype == TPB200_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + e0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float4 t = __ldg(p + i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + e0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 t = __ldg(p + i);
            const uint32_t u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float2 f;
                if (x_dtype == TPB200_F16) {
                    f = __half22float2(*reinterpret_cast<const __half2*>(&u[q]));
                } else {
                    f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[q]));
                }
                v[8 * i + 2 * q] = f.x;
                v[8 * i + 2 * q + 1] = f.y;
            }
        }
    }
    if (xs != nullptr) {  // per-block activation scales, dtype of x
        const size_t per_row = row_off / group;  // row_off = m*K, K % group == 0
        if (group == 16) {
            float s0 = load_as_float(xs, x_dtype, per_row + 2 * static_cast<size_t>(j));
            float s1 = load_as_float(xs, x_dtype, per_row + 2 * static_cast<size_t>(j) + 1);
#pragma unroll
            for (int i = 0; i < 16; ++i) { v[i] *= s0; v[16 + i] *= s1; }
        } else {
            float s0 = load_as_float(xs, x_dtype, per_row + (static_cast<size_t>(j) * 32) / group);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= s0;
        }
    }
    if (prescale != 1.0f) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= prescale;
    }
    if (FMT == kFmtE2M1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) xr[i] = __halves2half2(to_half_sat(v[2 * i]), to_half_sat(v[2 * i + 1]));
    } else {
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                xr[wd * 4 + p] = __halves2half2(to_half_sat(v[8 * wd + p]), to_half_sat(v[8 * wd + p + 4]));
            }
        }
    }
}

template <int SCALE_MODE>
__device__ __forceinline__ void load_chunk_scales(const uint8_t* sc_row, int j, int group, float& s0, float& s1) {
    if (SCALE_MODE == kScE4M3B16) {
        float2 f = decode_e4m3x2(*reinterpret_cast<const uint16_t*>(sc_row + 2 * j));
        s0 = f.x; s1 = f.y;
    } else if (SCALE_MODE == kScE4M3B32) {
        s0 = s1 = decode_e4m3(sc_row[j]);
    } else if (SCALE_MODE == kScF32B16) {
        float2 f = *reinterpret_cast<const float2*>(sc_row + 8 * j);
        s0 = f.x; s1 = f.y;
    } else if (SCALE_MODE == kScF32B32) {
        s0 = s1 = *reinterpret_cast<const float*>(sc_row + 4 * j);
    } else if (SCALE_MODE == kScF16Group) {
        s0 = s1 = __half2float(reinterpret_cast<const __half*>(sc_row)[(j * 32) / group]);
    } else {
        s0 = s1 = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(sc_row)[(j * 32) / group]);
    }
}

// sum over 16 codes (two words) of code * x as a packed fp16 pair (even/odd lanes of the
// pairing still separate): two chains of four products, added at the end
__device__ __forceinline__ __half2 dot16h(const __half2 (&ha)[4], const __half2 (&hb)[4], const __half2* x) {
    __half2 a = __hmul2(ha[0], x[0]);
    __half2 b = __hmul2(hb[0], x[4]);
    a = __hfma2(ha[1], x[1], a);
    b = __hfma2(hb[1], x[5], b);
    a = __hfma2(ha[2], x[2], a);
    b = __hfma2(hb[2], x[6], b);
    a = __hfma2(ha[3], x[3], a);
    b = __hfma2(hb[3], x[7], b);
    return __hadd2(a, b);
}

__device__ __forceinline__ float hsum2(__half2 v) {
    const float2 f = __half22float2(v);
    return f.x + f.y;
}

// E4M3 block scales are exact in fp16, so the two 16-code sums of a chunk are scaled and added
// in packed fp16 and widened once.  To keep sum * scale (scale up to 448) inside fp16 range the
// activations of these modes are stored pre-multiplied by 2^-8 (kXPrescale) and the result is
// multiplied back in the epilogue.
constexpr float kXPrescale = 1.0f / 256.0f;
template <int SCALE_MODE>
__host__ __device__ constexpr bool scales_in_half() { return SCALE_MODE == kScE4M3B16 || SCALE_MODE == kScE4M3B32; }

template <int SCALE_MODE>
__device__ __forceinline__ void load_chunk_scales_h2(const uint8_t* sc_row, int j, __half2& s0, __half2& s1) {
    uint32_t r;
    if (SCALE_MODE == kScE4M3B16) {
        const uint16_t v = *reinterpret_cast<const uint16_t*>(sc_row + 2 * j);
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    } else {
        const uint16_t v = static_cast<uint16_t>(sc_row[j]) * 0x0101u;
        asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    }
    const __half2 h = *reinterpret_cast<__half2*>(&r);
    s0 = __low2half2(h);
    s1 = __high2half2(h);
}

// Sum four per-lane values over the warp at once: after the call lane 8*i (i = 0..3) holds the
// warp total of v[i].  6 shuffles instead of 20.
__device__ __forceinline__ float warp_sum4(const float (&v)[4], int lane) {
    const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0;
    float k0 = b4 ? v[2] : v[0];
    float k1 = b4 ? v[3] : v[1];
    const float s0 = b4 ? v[0] : v[2];
    const float s1 = b4 ? v[1] : v[3];
    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
    float k = b3 ? k1 : k0;
    const float sx = b3 ? k0 : k1;
    k += __shfl_xor_sync(0xffffffffu, sx, 8);
    k += __shfl_xor_sync(0xffffffffu, k, 4);
    k += __shfl_xor_sync(0xffffffffu, k, 2);
    k += __shfl_xor_sync(0xffffffffu, k, 1);
    return k;
}

// Per-lane partial sums of one group of RG = 4 / M_TILE rows (rbase, rbase + RW, ...) over the
// lane's chunk columns of K-part `kp`: acc[g * M_TILE + m].
template <int FMT, int SCALE_MODE, int M_TILE, int CPL>
__device__ __forceinline__ void accumulate_row_group(float (&acc)[4], const __half2 (&xr)[M_TILE][CPL][16],
                                                     const uint8_t* wt, const uint8_t* sc, int row_bytes,
                                                     int scale_row_bytes, int rbase, int RW, int rows, int kp,
                                                     int lane, int nchunks, int group, uint32_t u4_xor) {
    constexpr int RG = 4 / M_TILE;
    acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
#pragma unroll
    for (int g = 0; g < RG; ++g) {
        const int r = rbase + g * RW;
        if (r < rows) {
#pragma unroll
            for (int c = 0; c < CPL; ++c) {
                const int j = (kp * CPL + c) * 32 + lane;
                if (j < nchunks) {
                    const uint4 w = *reinterpret_cast<const uint4*>(wt + r * row_bytes + j * 16);
                    const uint8_t* sc_row = sc + static_cast<size_t>(r) * scale_row_bytes;
                    __half2 h0[4], h1[4], h2[4], h3[4];
                    if (FMT == kFmtE2M1) {
                        decode_e2m1x8(w.x, h0); decode_e2m1x8(w.y, h1);
                        decode_e2m1x8(w.z, h2); decode_e2m1x8(w.w, h3);
                    } else {
                        decode_u4x8_minus8(w.x ^ u4_xor, h0); decode_u4x8_minus8(w.y ^ u4_xor, h1);
                        decode_u4x8_minus8(w.z ^ u4_xor, h2); decode_u4x8_minus8(w.w ^ u4_xor, h3);
                    }
                    if (scales_in_half<SCALE_MODE>()) {
                        __half2 s0, s1;
                        load_chunk_scales_h2<SCALE_MODE>(sc_row, j, s0, s1);
#pragma unroll
                        for (int m = 0; m < M_TILE; ++m) {
                            const __half2 d0 = dot16h(h0, h1, &xr[m][c][0]);
                            const __half2 d1 = dot16h(h2, h3, &xr[m][c][8]);
                            acc[g * M_TILE + m] += hsum2(__hfma2(d0, s0, __hmul2(d1, s1)));
                        }
                    } else {
                        float s0, s1;
                        load_chunk_scales<SCALE_MODE>(sc_row, j, group, s0, s1);
#pragma unroll
                        for (int m = 0; m < M_TILE; ++m) {
                            const float d0 = hsum2(dot16h(h0, h1, &xr[m][c][0]));
                            const float d1 = hsum2(dot16h(h2, h3, &xr[m][c][8]));
                            acc[g * M_TILE + m] = fmaf(d0, s0, acc[g * M_TILE + m]);
                            acc[g * M_TILE + m] = fmaf(d1, s1, acc[g * M_TILE + m]);
                        }
                    }
                }
            }
        }
    }
}

template <int FMT, int SCALE_MODE, int M_TILE, int CPL, int MAXP>
__global__ void __launch_bounds__(kThreads, 2) gemv_rowmajor_kernel(const __grid_constant__ GemvParams<MAXP> P) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* wst = smem;
    uint8_t* sst = smem + kStages * kWStage;
    float* part = reinterpret_cast<float*>(sst + kStages * kSStage);
    uint64_t* full = reinterpret_cast<uint64_t*>(part + 2 * kMaxPartials * M_TILE);
    int* abort_flag = reinterpret_cast<int*>(full + kStages);

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int total_tiles = P.total_tiles;
    const int m0 = blockIdx.y * M_TILE;
    const int group = P.group;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();

    // This CTA owns the contiguous tile range [tile_lo, tile_hi): consecutive tiles belong to the
    // same matrix, so the activation registers are reloaded only when the range crosses into
    // the next problem.
    const int tile_lo = static_cast<int>(static_cast<long long>(blockIdx.x) * total_tiles / gridDim.x);
    const int tile_hi = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * total_tiles / gridDim.x);

    // Producer (thread 0): request tile number `it` of this CTA.  `ip` follows the problem index.
    int ip = find_problem(P, tile_lo);
    auto issue = [&](int it) {
        const int tile = tile_lo + it;
        if (tile >= tile_hi) return;
        while (ip + 1 < P.num_problems && tile >= P.prob[ip + 1].tile_begin) ++ip;
        const ProblemDev& pr = P.prob[ip];
        const int row0 = (tile - pr.tile_begin) * pr.rows_per_tile;
        const int rows = min(pr.rows_per_tile, pr.N - row0);
        const int row_bytes = pr.K >> 1;
        const int s = it % kStages;
        const uint32_t wbytes = static_cast<uint32_t>(rows) * row_bytes;
        const uint32_t sbytes = pr.scales_by_tma ? static_cast<uint32_t>(rows) * pr.scale_row_bytes : 0u;
        mbar_expect_tx(&full[s], wbytes + sbytes);
        bulk_copy_g2s_hint(wst + s * kWStage, pr.w + static_cast<size_t>(row0) * row_bytes, wbytes, &full[s], l2_policy_evict_first());
        if (sbytes) {
            bulk_copy_g2s(sst + s * kSStage, pr.scales + static_cast<size_t>(row0) * pr.scale_row_bytes, sbytes,
                          &full[s]);
        }
    };
    if (tid == 0) {
#pragma unroll
        for (int it = 0; it < kStages; ++it) issue(it);
    }
    // Weights are in flight; let the next kernel start its own prefetch, then wait
    // for whatever produced our activations (and last read our output buffer).
    pdl_launch_dependents();
    pdl_wait_prior_grids();

    __half2 xr[M_TILE][CPL][16];
    int p = find_problem(P, tile_lo), cur_p = -1;
    int KP = 1, kp = 0, rw = 0, RW = kWarps, nchunks = 0;

    for (int it = 0;; ++it) {
        const int tile = tile_lo + it;
        if (tile >= tile_hi) break;
        while (p + 1 < P.num_problems && tile >= P.prob[p + 1].tile_begin) ++p;
        const ProblemDev& pr = P.prob[p];
        if (p != cur_p) {
            cur_p = p;
            KP = pr.kparts;
            RW = kWarps / KP;
            kp = warp % KP;
            rw = warp / KP;
            nchunks = pr.K >> 5;
#pragma unroll
            for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
                for (int c = 0; c < CPL; ++c) {
                    const int j = (kp * CPL + c) * 32 + lane;
                    load_x_chunk<FMT>(xr[m][c], pr.x, pr.x_scales, P.x_dtype,
                                      static_cast<size_t>(m0 + m) * pr.K, j, group,
                                      (j < nchunks) && (m0 + m < P.M),
                                      scales_in_half<SCALE_MODE>() ? kXPrescale : 1.0f);
                }
            }
        }
        const int row0 = (tile - pr.tile_begin) * pr.rows_per_tile;
        const int rows = min(pr.rows_per_tile, pr.N - row0);
        const int row_bytes = pr.K >> 1;
        const int s = it % kStages;
        if (!mbar_wait_bounded(&full[s], (it / kStages) & 1)) {
            record_error(kErrGemvFullBarrierTimeout);
            *abort_flag = 1;
        }
        const uint8_t* wt = wst + s * kWStage;
        const uint8_t* sc = pr.scales_by_tma ? (sst + s * kSStage)
                                             : (pr.scales + static_cast<size_t>(row0) * pr.scale_row_bytes);
        float* pt = part + (it & 1) * kMaxPartials * M_TILE;

        // Each warp takes its rows (rw, rw + RW, ...) in groups of RG = 4 / M_TILE, so that the four
        // (row, m) sums of a group are reduced over the warp together.
        constexpr int RG = 4 / M_TILE;
        for (int rbase = rw; rbase < rows; rbase += RW * RG) {
            float acc[4];
            accumulate_row_group<FMT, SCALE_MODE, M_TILE, CPL>(acc, xr, wt, sc, row_bytes, pr.scale_row_bytes, rbase, RW,
                                                               rows, kp, lane, nchunks, group, P.u4_xor);
            const float total = warp_sum4(acc, lane);
            if ((lane & 7) == 0) {
                const int idx = lane >> 3;
                const int r = rbase + (idx / M_TILE) * RW;
                if (r < rows) pt[(r * KP + kp) * M_TILE + (idx % M_TILE)] = total;
            }
        }
        __syncthreads();  // partial sums visible; every thread is done with stage s
        if (*abort_flag) break;
        if (tid == 0) issue(it + kStages);
        if (tid < rows * M_TILE) {
            const int m = tid / rows;
            const int r = tid - m * rows;
            if (m0 + m < P.M) {
                float v = 0.0f;
                for (int q = 0; q < KP; ++q) v += pt[(r * KP + q) * M_TILE + m];
                v *= scales_in_half<SCALE_MODE>() ? pr.global_scale * (1.0f / kXPrescale) : pr.global_scale;
                if (pr.bias != nullptr) v += load_as_float(pr.bias, P.bias_dtype, row0 + r);
                v = apply_activation(v, P.activation);
                store_from_float(pr.out, P.out_dtype, static_cast<size_t>(m0 + m) * pr.ldo + row0 + r, v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Warp-specialised variant for launches in which no row is split across warps (every problem has
// kparts == 1, i.e. K <= 1024 * CPL): eight consumer warps and one producer warp per CTA, and no
// CTA-wide barrier in the tile loop.  The producer lane refills a stage as soon as all eight
// consumer warps have released it (an `empty` mbarrier per stage), so warps drift apart freely;
// each warp reduces and stores its own rows.
// ---------------------------------------------------------------------------------------------
constexpr int kWsThreads = kThreads + 32;

template <int FMT, int SCALE_MODE, int M_TILE, int CPL, int MAXP>
__global__ void __launch_bounds__(kWsThreads, 2) gemv_rowmajor_ws_kernel(const __grid_constant__ GemvParams<MAXP> P) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* wst = smem;
    uint8_t* sst = smem + kStages * kWStage;
    uint64_t* full = reinterpret_cast<uint64_t*>(sst + kStages * kSStage);
    uint64_t* empty = full + kStages;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int total_tiles = P.total_tiles;
    const int m0 = blockIdx.y * M_TILE;
    const int group = P.group;
    const int tile_lo = static_cast<int>(static_cast<long long>(blockIdx.x) * total_tiles / gridDim.x);
    const int tile_hi = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * total_tiles / gridDim.x);

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], kWarps);
        }
        fence_mbar_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == kWarps) {
        // ---------------- producer: one lane streams this CTA's tiles through the ring ----------------
        if (lane == 0) {
            int ip = find_problem(P, tile_lo);
            for (int it = 0; tile_lo + it < tile_hi; ++it) {
                const int tile = tile_lo + it;
                const int s = it % kStages;
                if (it >= kStages && !mbar_wait_bounded(&empty[s], ((it / kStages) - 1) & 1)) {
                    record_error(kErrGemvEmptyBarrierTimeout);
                    break;
                }
                while (ip + 1 < P.num_problems && tile >= P.prob[ip + 1].tile_begin) ++ip;
                const ProblemDev& pr = P.prob[ip];
                const int row0 = (tile - pr.tile_begin) * pr.rows_per_tile;
                const int rows = min(pr.rows_per_tile, pr.N - row0);
                const int row_bytes = pr.K >> 1;
                const uint32_t wbytes = static_cast<uint32_t>(rows) * row_bytes;
                const uint32_t sbytes = pr.scales_by_tma ? static_cast<uint32_t>(rows) * pr.scale_row_bytes : 0u;
                mbar_expect_tx(&full[s], wbytes + sbytes);
                bulk_copy_g2s_hint(wst + s * kWStage, pr.w + static_cast<size_t>(row0) * row_bytes, wbytes, &full[s], l2_policy_evict_first());
                if (sbytes) {
                    bulk_copy_g2s(sst + s * kSStage, pr.scales + static_cast<size_t>(row0) * pr.scale_row_bytes,
                                  sbytes, &full[s]);
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    pdl_wait_prior_grids();  // activations and the output buffer belong to earlier kernels until here
    __half2 xr[M_TILE][CPL][16];
    int p = find_problem(P, tile_lo), cur_p = -1, nchunks = 0;
    constexpr int RG = 4 / M_TILE;
    for (int it = 0; tile_lo + it < tile_hi; ++it) {
        const int tile = tile_lo + it;
        while (p + 1 < P.num_problems && tile >= P.prob[p + 1].tile_begin) ++p;
        const ProblemDev& pr = P.prob[p];
        if (p != cur_p) {
            cur_p = p;
            nchunks = pr.K >> 5;
#pragma unroll
            for (int m = 0; m < M_TILE; ++m) {
#pragma unroll
                for (int c = 0; c < CPL; ++c) {
                    const int j = c * 32 + lane;
                    load_x_chunk<FMT>(xr[m][c], pr.x, pr.x_scales, P.x_dtype, static_cast<size_t>(m0 + m) * pr.K, j,
                                      group, (j < nchunks) && (m0 + m < P.M),
                                      scales_in_half<SCALE_MODE>() ? kXPrescale : 1.0f);
                }
            }
        }
        const int row0 = (tile - pr.tile_begin) * pr.rows_per_tile;
        const int rows = min(pr.rows_per_tile, pr.N - row0);
        const int row_bytes = pr.K >> 1;
        const int s = it % kStages;
        if (!mbar_wait_bounded(&full[s], (it / kStages) & 1)) {
            record_error(kErrGemvFullBarrierTimeout);
            break;
        }
        const uint8_t* wt = wst + s * kWStage;
        const uint8_t* sc = pr.scales_by_tma ? (sst + s * kSStage)
                                             : (pr.scales + static_cast<size_t>(row0) * pr.scale_row_bytes);
        const float out_scale = scales_in_half<SCALE_MODE>() ? pr.global_scale * (1.0f / kXPrescale) : pr.global_scale;
        for (int rbase = warp; rbase < rows; rbase += kWarps * RG) {
            float acc[4];
            accumulate_row_group<FMT, SCALE_MODE, M_TILE, CPL>(acc, xr, wt, sc, row_bytes, pr.scale_row_bytes, rbase,
                                                               kWarps, rows, 0, lane, nchunks, group, P.u4_xor);
            float v = warp_sum4(acc, lane);
            if ((lane & 7) == 0) {
                const int idx = lane >> 3;
                const int r = rbase + (idx / M_TILE) * kWarps;
                const int m = idx % M_TILE;
                if (r < rows && m0 + m < P.M) {
                    v *= out_scale;
                    if (pr.bias != nullptr) v += load_as_float(pr.bias, P.bias_dtype, row0 + r);
                    v = apply_activation(v, P.activation);
                    store_from_float(pr.out, P.out_dtype, static_cast<size_t>(m0 + m) * pr.ldo + row0 + r, v);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);  // this warp is done reading stage s
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct HostProblem {
    const void* x;
    const void* x_scales;
    const void* w;
    const void* scales;
    const void* bias;
    void* out;
    int N, K;
    float global_scale;
    int ldo = 0;   // 0: rows of `out` are N apart
};

struct Plan {
    int m_tile, cpl, kparts;
};

// Choose the M tile, K-parts and chunk columns per lane for the LARGEST K of the launch
// (M_TILE * CPL <= 4 keeps the activation registers within 64).
bool make_plan(int M, int maxK, Plan& plan) {
    int m_tile = M >= 3 ? 4 : M;
    const int nchunks = maxK / 32;
    while (m_tile >= 1) {
        const int cplmax = 4 / m_tile;
        int kparts = 1;
        while ((nchunks + 32 * kparts - 1) / (32 * kparts) > cplmax && kparts < 8) kparts *= 2;
        const int need = (nchunks + 32 * kparts - 1) / (32 * kparts);
        if (need <= cplmax) {
            plan.m_tile = m_tile;
            plan.cpl = need <= 1 ? 1 : (need <= 2 ? 2 : 4);
            plan.kparts = kparts;
            return true;
        }
        m_tile /= 2;
    }
    return false;
}

template <typename Kernel, typename Params>
int launch_kernel(Kernel kernel, const Params& P, int threads, size_t smem, std::atomic<uint64_t>& configured,
                  int grid_x, int grid_y, int flags, cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return TPB200_ERR_CUDA;
    const uint64_t bit = 1ull << (dev & 63);  // bit d: attribute set on device d
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
            cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid_x, grid_y, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, kernel, P) != cudaSuccess) return TPB200_ERR_CUDA;
    return TPB200_OK;
}

template <int FMT, int SCALE_MODE, int M_TILE, int CPL, int MAXP>
int launch_instance(const GemvParams<MAXP>& P, bool warp_specialised, int grid_x, int grid_y, int flags,
                    cudaStream_t stream) {
    if (warp_specialised) {
        static std::atomic<uint64_t> configured_ws{0};
        const size_t smem = kStages * (kWStage + kSStage) + 2 * kStages * sizeof(uint64_t);
        return launch_kernel(gemv_rowmajor_ws_kernel<FMT, SCALE_MODE, M_TILE, CPL, MAXP>, P, kWsThreads, smem,
                             configured_ws, grid_x, grid_y, flags, stream);
    }
    static std::atomic<uint64_t> configured{0};
    const size_t smem = kStages * (kWStage + kSStage) + 2 * kMaxPartials * M_TILE * sizeof(float) +
                        kStages * sizeof(uint64_t) + 16;
    return launch_kernel(gemv_rowmajor_kernel<FMT, SCALE_MODE, M_TILE, CPL, MAXP>, P, kThreads, smem, configured,
                         grid_x, grid_y, flags, stream);
}

template <int FMT, int SCALE_MODE, int MAXP>
int dispatch_tiles(const GemvParams<MAXP>& P, const Plan& plan, bool ws, int grid_x, int grid_y, int flags,
                   cudaStream_t stream) {
#define TPB_CASE(MT, C)                              \
    if (plan.m_tile == MT && plan.cpl == C)          \
        return launch_instance<FMT, SCALE_MODE, MT, C, MAXP>(P, ws, grid_x, grid_y, flags, stream);
    TPB_CASE(1, 1) TPB_CASE(1, 2) TPB_CASE(1, 4) TPB_CASE(2, 1) TPB_CASE(2, 2) TPB_CASE(4, 1)
#undef TPB_CASE
    return TPB200_ERR_SHAPE;
}

template <int MAXP>
int run_gemv(int fmt_in, const HostProblem* probs, int count, int x_dtype, int scale_dtype, int group,
             int bias_dtype, int out_dtype, int M, int activation, int flags, cudaStream_t stream) {
    const int fmt = fmt_in == 2 ? kFmtU4 : fmt_in;   // 2 = signed (two's complement) int4
    TPB_REQUIRE(probs != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= MAXP, TPB200_ERR_SHAPE);
    TPB_REQUIRE(M >= 1 && M <= 16, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(x_dtype) && tpb_valid_dtype(out_dtype) && tpb_valid_dtype(bias_dtype),
                TPB200_ERR_ENUM);
    TPB_REQUIRE(activation >= TPB200_ACT_NONE && activation <= TPB200_ACT_SILU, TPB200_ERR_ENUM);
    TPB_REQUIRE((flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    int scale_mode, scale_bytes;
    if (fmt == kFmtE2M1) {
        TPB_REQUIRE(group == 16 || group == 32, TPB200_ERR_SHAPE);
        if (scale_dtype == TPB200_SCALE_E4M3) {
            scale_mode = group == 16 ? kScE4M3B16 : kScE4M3B32;
            scale_bytes = 1;
        } else if (scale_dtype == TPB200_SCALE_F32) {
            scale_mode = group == 16 ? kScF32B16 : kScF32B32;
            scale_bytes = 4;
        } else {
            return TPB200_ERR_ENUM;
        }
    } else {
        TPB_REQUIRE(group >= 32 && group % 32 == 0, TPB200_ERR_SHAPE);
        if (scale_dtype == TPB200_SCALE_F16) scale_mode = kScF16Group;
        else if (scale_dtype == TPB200_SCALE_BF16) scale_mode = kScBF16Group;
        else return TPB200_ERR_ENUM;
        scale_bytes = 2;
    }

    int maxK = 0;
    for (int i = 0; i < count; ++i) {
        const HostProblem& h = probs[i];
        TPB_REQUIRE(h.x && h.w && h.scales && h.out, TPB200_ERR_NULL);
        TPB_REQUIRE(h.N >= 1 && h.K >= 32 && h.K % 32 == 0 && h.K % group == 0, TPB200_ERR_SHAPE);
        TPB_REQUIRE(h.ldo == 0 || h.ldo >= h.N, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(h.x) && tpb_aligned16(h.w) && tpb_aligned16(h.scales) && tpb_aligned16(h.out),
                    TPB200_ERR_ALIGN);
        maxK = std::max(maxK, h.K);
    }
    Plan plan;
    TPB_REQUIRE(make_plan(M, maxK, plan), TPB200_ERR_SHAPE);

    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }

    GemvParams<MAXP> P;
    P.num_problems = count;
    P.M = M;
    P.x_dtype = x_dtype;
    P.bias_dtype = bias_dtype;
    P.out_dtype = out_dtype;
    P.activation = activation;
    P.group = group;
    P.u4_xor = fmt_in == 2 ? 0x88888888u : 0u;
    long long weight_bytes = 0;
    for (int i = 0; i < count; ++i) weight_bytes += static_cast<long long>(probs[i].N) * (probs[i].K / 2);
    const long long target_tile_bytes =
        std::min<long long>(kWStage, std::max<long long>(4096, weight_bytes / (16LL * sms)));
    int tiles = 0;
    for (int i = 0; i < count; ++i) {
        const HostProblem& h = probs[i];
        ProblemDev& d = P.prob[i];
        d.w = static_cast<const uint8_t*>(h.w);
        d.scales = static_cast<const uint8_t*>(h.scales);
        d.x = h.x;
        d.x_scales = h.x_scales;
        d.bias = h.bias;
        d.out = h.out;
        d.N = h.N;
        d.K = h.K;
        d.ldo = h.ldo > 0 ? h.ldo : h.N;
        d.global_scale = h.global_scale;
        // K-parts for THIS problem under the launch-wide CPL
        const int nchunks = h.K / 32;
        int kparts = 1;
        while ((nchunks + 32 * kparts - 1) / (32 * kparts) > plan.cpl && kparts < 8) kparts *= 2;
        d.kparts = kparts;
        const int rw = kWarps / kparts;
        const int row_bytes = h.K / 2;
        d.scale_row_bytes = (h.K / group) * scale_bytes;
        int rmax = std::min({kMaxTileRows, kWStage / row_bytes, kMaxPartials / kparts});
        rmax = std::max(rw, rmax / rw * rw);
        TPB_REQUIRE(rmax * row_bytes <= kWStage, TPB200_ERR_SHAPE);
        // tile bytes: the whole launch split into ~8 tiles per CTA (2 CTAs per SM), within 4..16 KB,
        // and at least one row per row-warp
        const int target_rows = static_cast<int>(target_tile_bytes / row_bytes) / rw * rw;
        int R = std::min(rmax, std::max(rw, target_rows));
        d.scales_by_tma = (d.scale_row_bytes % 16 == 0) && (R * d.scale_row_bytes <= kSStage) ? 1 : 0;
        d.rows_per_tile = R;
        d.tile_begin = tiles;
        tiles += (h.N + R - 1) / R;
    }
    P.total_tiles = tiles;
    bool ws = true;  // no row split across warps anywhere in the launch -> warp-specialised kernel
    for (int i = 0; i < count; ++i) ws = ws && (P.prob[i].kparts == 1);
    const int grid_x = std::min(tiles, 2 * sms);
    const int grid_y = (M + plan.m_tile - 1) / plan.m_tile;

#define TPB_MODE(F, S) \
    if (fmt == F && scale_mode == S) return dispatch_tiles<F, S, MAXP>(P, plan, ws, grid_x, grid_y, flags, stream);
    TPB_MODE(kFmtE2M1, kScE4M3B16)
    TPB_MODE(kFmtE2M1, kScF32B32)
    if (MAXP == 1) {
        TPB_MODE(kFmtE2M1, kScE4M3B32)
        TPB_MODE(kFmtE2M1, kScF32B16)
        TPB_MODE(kFmtU4, kScF16Group)
        TPB_MODE(kFmtU4, kScBF16Group)
    }
#undef TPB_MODE
    return TPB200_ERR_ENUM;
}

}  // namespace

int gemv_rowmajor_single(int fmt_is_u4, const void* x, int x_dtype, const void* x_scales, const void* w,
                         const void* scales, int scale_dtype, int group, float global_scale, const void* bias,
                         int bias_dtype, void* out, int out_dtype, int M, int N, int K, int activation, int flags,
                         cudaStream_t stream) {
    HostProblem h{x, x_scales, w, scales, bias, out, N, K, global_scale};
    return run_gemv<1>(fmt_is_u4 == 2 ? 2 : (fmt_is_u4 ? kFmtU4 : kFmtE2M1), &h, 1, x_dtype, scale_dtype, group, bias_dtype, out_dtype, M,
                       activation, flags, stream);
}

int device_error_gemv_rowmajor(int clear) { return read_device_error(clear); }

}  // namespace tpb

extern "C" int tpb200_nvfp4_gemv(const void* x, int x_dtype, const void* x_scales, const void* weight_packed,
                                 const void* weight_scales, int scale_dtype, int block_size, float global_scale,
                                 const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K,
                                 int activation, int flags, tpb200_stream_t stream) {
    return tpb::gemv_rowmajor_single(0, x, x_dtype, x_scales, weight_packed, weight_scales, scale_dtype, block_size,
                                     global_scale, bias, bias_dtype, out, out_dtype, M, N, K, activation, flags,
                                     reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tpb200_nvfp4_gemv_grouped(const tpb200_gemv_problem* problems, int count, int x_dtype,
                                         int scale_dtype, int block_size, int bias_dtype, int out_dtype, int M,
                                         int activation, int flags, tpb200_stream_t stream) {
    TPB_REQUIRE(problems != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_GROUP, TPB200_ERR_SHAPE);
    tpb::HostProblem h[TPB200_MAX_GROUP];
    for (int i = 0; i < count; ++i) {
        h[i] = tpb::HostProblem{problems[i].x, nullptr, problems[i].weight_packed, problems[i].weight_scales,
                                problems[i].bias, problems[i].out, problems[i].N, problems[i].K,
                                problems[i].global_scale, problems[i].out_stride};
    }
    return tpb::run_gemv<TPB200_MAX_GROUP>(tpb::kFmtE2M1, h, count, x_dtype, scale_dtype, block_size, bias_dtype,
                                           out_dtype, M, activation, flags, reinterpret_cast<cudaStream_t>(stream));
}
