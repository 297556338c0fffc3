// NVFP4 x NVFP4 block-scaled GEMM on the 5th-generation tensor cores:
//   out[M, N] = act(alpha * rowscale[m] * sum_p sum_k (a_p[m,k] * sfa_p[m,k/16]) * (b[n,k] * sfb[n,k/16]) + bias[n])
// a_p, b: e2m1 codes, two per byte (even k in the low nibble), K-major; sfa, sfb: UE4M3 per 16
// along K, stored in 512-byte atoms of 128 rows x 4 K-blocks (byte (r%32)*16 + (r/32)*4 + kb),
// atoms ordered [row tile][K atom].  The A operand may consist of up to four residual pieces
// (weight-only semantics for bf16 activations); all pieces of a K stage are multiplied against
// ONE resident B tile.
//
// One persistent CTA per SM, warp-specialised:
//   warp 0     TMA producer: per 256-wide K stage one 128B-swizzled box of B (128 rows), one per
//              A piece, and their 2 KB scale slabs (plain bulk copies), ring of 2..5 stages;
//   warp 1     allocates tensor memory; one lane copies the stage's scale atoms shared->tensor
//              memory (tcgen05.cp) and issues 4 tcgen05.mma kind::mxf4nvf4 (K = 64 each) per piece
//              into one of two 128x128 fp32 accumulators, committing the stage back to the producer;
//   warps 2-5  epilogue: tcgen05.ld, alpha / row scale / bias / activation (or rotary embedding for
//              the fused QKV form), conversion, 128B-swizzled staging in shared memory and TMA
//              tile stores (full-line writes, clipped at the matrix edge by the tensor map).
// One CTA per SM, no clusters: no operand is shared between CTAs; every wait is bounded and reports
// through the device error word.
//
// Two operand formats.  Row-major (the reference's): tiles of 128 x 128 outputs, operands fetched with
// tiled TMA boxes.  Tiled images (kTiled): both operands pre-arranged so that everything one K stage
// needs from an operand is ONE contiguous block -- B block (n_blk, ks) = 256 rows x 128 B of codes in
// the 128B-swizzle pattern + their two scale slabs (36 KB), A block (m_blk, ks) = the code tiles of all
// pieces + their scale slabs (18 KB per piece) -- fetched with two plain bulk copies per stage into
// tiles of 128 x 256 outputs.  An SM takes in roughly 0.3 us per copy request whatever its size (the
// measured rate grows from ~25 GB/s with 8 KB requests to ~100 GB/s with 32 KB+), and this kernel is
// bound by exactly that intake, so the tiled form both halves the bytes per flop (B shared by twice
// the columns) and moves them in requests of 36-54 KB instead of 2-16 KB.
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "tcgen05.cuh"

namespace tpb {
namespace {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;            // 256 e2m1 codes per row per stage
constexpr int kMaxStages = 5;
constexpr int kMaxPieces = 4;
constexpr int kTile = 128 * kBKBytes;    // 16 KB operand tile
constexpr int kSfSlab = 4 * 512;         // 4 K-atoms of one 128-row tile
constexpr int kOutBuf = 128 * 128;       // one staged output box: 128 rows x 128 bytes
constexpr int kThreads = 320;           // warps: 0 producer, 1 MMA issuer, 2..5 and 6..9 two epilogue groups
constexpr int kTmemCols = 512;
// tensor memory: columns [0, 256) hold two 128-column accumulators (row-major form) or one of 256
// columns (tiled form); then the B scales (4 columns per K atom and 128 rows) and 16 columns per A piece
constexpr uint32_t kSfbCol = 256;
constexpr uint32_t kSfaCol = kSfbCol + 32;
constexpr int kSmemBudget = 227 * 1024 - 2048;
constexpr int kBlock = kTile + kSfSlab;  // codes + scales of 128 rows for one K stage (18 KB)

__host__ __device__ constexpr int tile_n(bool tiled) { return tiled ? 256 : 128; }
__host__ __device__ constexpr int stage_bytes(int pieces, bool tiled) { return ((tiled ? 2 : 1) + pieces) * kBlock; }
__host__ __device__ constexpr int num_stages(int pieces, bool tiled) {
    return (kSmemBudget - 2 * kOutBuf) / stage_bytes(pieces, tiled) < kMaxStages
               ? (kSmemBudget - 2 * kOutBuf) / stage_bytes(pieces, tiled)
               : kMaxStages;
}

struct alignas(64) GemmParams {
    CUtensorMap map_a;
    CUtensorMap map_b;
    CUtensorMap map_out;       // plain epilogue: out; fused QKV: q_out
    CUtensorMap map_k;         // fused QKV: K cache rows
    CUtensorMap map_v;         // fused QKV: V cache rows
    const uint8_t* sfa;
    const uint8_t* sfb;
    const uint8_t* a_image;    // tiled form: blocks [m_blk][ks] of pieces * 18 KB
    const uint8_t* b_image;    // tiled form: blocks [n_blk][ks] of 36 KB
    const float* bias;
    int M, N, K;
    int out_dtype;
    int activation;
    float alpha;
    int k_stages;   // ceil(K / 256)
    int m_blocks, n_blocks;
    // A operand given as `a_pieces` residual pieces stacked along rows (piece p at row p * a_piece_rows)
    int a_pieces;
    int a_piece_rows;
    const float* row_scale;  // optional per-row multiplier of the result (undoes the activation pre-scale)
    // fused QKV epilogue (epilogue == kEpiQkvRope): rotary embedding on the Q and K heads, K/V rows
    // appended to the cache.  B rows are stored tile-permuted: tile t = 2 * head + half holds
    // head rows [64*half, 64*half + 64) followed by their rotation partners (+128).
    int epilogue;
    int q_dim;                 // number of Q outputs (heads * 256); then 256 K and 256 V outputs
    const int* positions;      // [M] index into the rotary tables
    const __nv_bfloat16* rope_cos;   // [positions, 128]
    const __nv_bfloat16* rope_sin;
    // split-K: work item w = tile * splits + split covers K stages [split * stages_per_split, ...);
    // partial accumulators go through `scratch` ([item][column / 4][row] float4); once all CTAs of a
    // tile have parked theirs, each finishes a slice of the tile's rows.
    int splits;
    int stages_per_split;
    float* scratch;
    unsigned int* counters;    // [2][kCounterSlots]: CTAs that parked their sums, CTAs that finished their slice
    // plain pointers for the split-K path's vector stores
    void* out;                 // plain: out; fused QKV: q_out
    int ldo;                   // elements
    __nv_bfloat16* k_rows;
    __nv_bfloat16* v_rows;
    int debug_slot;            // diagnostic builds: which timeline slot this launch writes
};
constexpr int kCounterSlots = 2048;

enum { kEpiPlain = 0, kEpiQkvRope = 1 };

struct SharedControl {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    alignas(16) float bias_s[2][128];  // the bias of the columns each epilogue group is working on
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// epilogue activations with the hardware approximations (results are rounded to bf16 anyway)
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    // 0.5 x (1 + tanh z) == x * sigmoid(2 z); this form has no cancellation for negative x
    const float z2 = 1.5957691216057308f * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-z2));
}
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void epilogue_group_barrier(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(1 + grp) : "memory"); }

// 16-byte chunk c of row r in a staged 128-byte-row box (the layout a 128B-swizzled TMA store reads)
__device__ __forceinline__ uint8_t* staged_chunk(uint8_t* buf, int r, int c) {
    return buf + r * 128 + ((c ^ (r & 7)) << 4);
}

// alpha / row scale, bias and activation on 32 consecutive outputs starting at column n
__device__ __forceinline__ void finish_plain32(float* v, float rs, const float* bias, int n, int N, int activation) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= rs;
    if (bias != nullptr) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            if (n + i < N) v[i] += __ldg(bias + n + i);
        }
    }
    // one uniform branch per chunk: the transcendental code stays out of the plain path
    if (activation == TPB200_ACT_GELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
    } else if (activation == TPB200_ACT_SILU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = silu_fast(v[i]);
    }
}

// the same with the 32 bias values already in shared memory (zeros past the end of the matrix, or no bias)
__device__ __forceinline__ void finish_plain32_staged(float* v, float rs, const float* bias_s, bool has_bias, int activation) {
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] *= rs;
    if (has_bias) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
            const float4 b = *reinterpret_cast<const float4*>(bias_s + i);
            v[i] += b.x; v[i + 1] += b.y; v[i + 2] += b.z; v[i + 3] += b.w;
        }
    }
    if (activation == TPB200_ACT_GELU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
    } else if (activation == TPB200_ACT_SILU) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = silu_fast(v[i]);
    }
}

// Gated GELU on 32 gate / up accumulator pairs, with the roundings of the module it replaces
// (GemmaMLP: down(act(gate(x)) * up(x)) on bf16 tensors): both projections rounded to bf16, the
// activation rounded to bf16, the product rounded by the store.
__device__ __forceinline__ void finish_geglu32(float* g, const float* u, float rs) {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float gb = __bfloat162float(__float2bfloat16_rn(g[i] * rs));
        const float ub = __bfloat162float(__float2bfloat16_rn(u[i] * rs));
        g[i] = __bfloat162float(__float2bfloat16_rn(gelu_tanh_fast(gb))) * ub;
    }
}

__device__ __forceinline__ void pack_bf16x32(const float* v, uint32_t* w) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&b2);
    }
}

// Rotary embedding on 32 head offsets (lo) and their partners 128 further on (hi), in bf16 as torch
// does it: x, cos, sin in bf16, each product and the sum rounded to bf16.  V heads pass through.
__device__ __forceinline__ void rope_pair32(const float* lo, const float* hi, float rs, const __nv_bfloat16* cos_row,
                                            const __nv_bfloat16* sin_row, bool is_v, uint32_t* olo, uint32_t* ohi) {
    const uint4* cs = reinterpret_cast<const uint4*>(cos_row);
    const uint4* sn = reinterpret_cast<const uint4*>(sin_row);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 cv = make_uint4(0, 0, 0, 0), sv = make_uint4(0, 0, 0, 0);
        if (!is_v) { cv = __ldg(cs + g); sv = __ldg(sn + g); }
        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = g * 8 + 2 * j;
            __nv_bfloat162 a = __floats2bfloat162_rn(lo[e] * rs, lo[e + 1] * rs);
            __nv_bfloat162 b = __floats2bfloat162_rn(hi[e] * rs, hi[e + 1] * rs);
            if (!is_v) {
                const __nv_bfloat162 co = *reinterpret_cast<const __nv_bfloat162*>(&cw[j]);
                const __nv_bfloat162 si = *reinterpret_cast<const __nv_bfloat162*>(&sw[j]);
                // first half: x*cos + (-x_partner)*sin ; second half: x_partner*cos + x*sin
                const __nv_bfloat162 ra = __hadd2(__hmul2(a, co), __hmul2(__hneg2(b), si));
                const __nv_bfloat162 rb = __hadd2(__hmul2(b, co), __hmul2(a, si));
                a = ra;
                b = rb;
            }
            olo[g * 4 + j] = *reinterpret_cast<uint32_t*>(&a);
            ohi[g * 4 + j] = *reinterpret_cast<uint32_t*>(&b);
        }
    }
}

#ifdef TPB_TIMELINE
// Diagnostic build only (-DTPB_TIMELINE): every CTA of the last launches leaves globaltimer stamps of its
// milestones here; tpb200_debug_gemm_timeline() copies them out.
constexpr int kTlSlots = 4, kTlPoints = 16, kTlCtas = 160;
__device__ unsigned long long g_gemm_timeline[kTlSlots][kTlCtas][kTlPoints];
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TL(point) g_gemm_timeline[P.debug_slot & (kTlSlots - 1)][blockIdx.x][point] = tl_now()
#else
#define TL(point) ((void)0)
#endif

template <bool kTiled>
__global__ void __launch_bounds__(kThreads, 1) nvfp4_gemm_kernel(const __grid_constant__ GemmParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int kBN = tile_n(kTiled);
    constexpr int kSubTiles = kBN / 128;          // 128-column halves of an output tile
    constexpr int kAccBufs = kTiled ? 1 : 2;
    constexpr int kItemFloat4 = 128 * kBN / 4;    // one parked partial accumulator
    const int pieces = P.a_pieces;
    const int nstages = num_stages(pieces, kTiled);
    const int stage_sz = stage_bytes(pieces, kTiled);
    // stage layout, row-major form: [B tile][A tile x pieces][SFB slab][SFA slab x pieces]
    //               tiled form:     [B 256 rows][SFB slab x 2][A tile x pieces][SFA slab x pieces]
    const int off_a = kTiled ? 2 * kBlock : kTile;
    const int off_sfb = kTiled ? 2 * kTile : (1 + pieces) * kTile;
    const int off_sfa = kTiled ? 2 * kBlock + pieces * kTile : off_sfb + kSfSlab;
    uint8_t* out_stage = smem + nstages * stage_sz;                       // 2 x 16 KB, 1024-byte aligned
    SharedControl* ctl = reinterpret_cast<SharedControl*>(out_stage + 2 * kOutBuf);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int splits = P.splits;
    const int total_items = P.m_blocks * P.n_blocks * splits;
    // Unsplit launches with the plain epilogue drain an accumulator with both epilogue groups (alternate
    // 128-byte boxes): the MMA thread waits for that drain before every tile, the accumulator being single.
    // The split-K hand-over and the fused QKV epilogue stay on group 0.
    const bool two_groups = P.epilogue == kEpiPlain && splits == 1;

    if (threadIdx.x == 0) {
        TL(0);
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], two_groups ? 8 : 4);   // one arrival per epilogue warp at work
        }
        ctl->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;
    if (threadIdx.x == 0) TL(1);
    // Programmatic dependent launch: everything above ran while the previous kernel of the stream may still
    // have been running.  The producer (operands) and the epilogue (row scales, bias, results, split-K
    // scratch) touch global memory, so they wait for it; the MMA issuer only ever sees shared memory.  The
    // producer first requests the WEIGHT halves of its first stages (tiled form): weights never depend on the
    // previous kernel, so their way from HBM overlaps that kernel's tail.
    pdl_launch_dependents();
    if (warp >= 2) pdl_wait_prior_grids();

    if (warp == 0) {
        // ------------------------------------------------------------ producer (whole warp).
        // Lane 0 owns the barrier hand-shakes; the stage's copy requests are issued by DIFFERENT lanes.  A
        // thread that issues a bulk copy is held for ~0.3 us whatever the size, so one lane issuing a stage's
        // requests back to back tops out near 60-90 GB/s per SM; the same requests issued side by side from
        // several lanes reach ~130 GB/s.  Tiled form: the stage is (2 + pieces) chunks of 18 KB, one per lane
        // (two from the B block, the rest from the contiguous A block).  Row-major form: one lane per box.
        if (!kTiled && lane == 0) {
            tc::prefetch_tensormap(&P.map_a);
            tc::prefetch_tensormap(&P.map_b);
        }
        const int sf_row_stride = P.k_stages * kSfSlab;   // bytes per 128-row tile of scales
        int s = 0;
        uint32_t empty_phase = 0;
        bool wrapped = false;                              // the first pass over the ring finds every stage free
        bool stop = false;
        int pre = 0;                                       // stages whose B half went out before the wait
        // weights are read once per inference (2.8 GB in all): they should not push the activations that the
        // next kernel reads out of L2
        const uint64_t weights_policy = l2_policy_evict_first();
        if (kTiled) {
            for (int w = blockIdx.x; w < total_items && pre < nstages; w += gridDim.x) {
                const int tile = w / splits;
                const int ks0 = (w - tile * splits) * P.stages_per_split;
                const int ks1 = min(P.k_stages, ks0 + P.stages_per_split);
                const int n_blk = tile / P.m_blocks;
                for (int ks = ks0; ks < ks1 && pre < nstages; ++ks, ++pre) {
                    if (lane == 0) mbar_expect_tx(&ctl->full[pre], stage_sz);
                    __syncwarp();
                    if (lane < 2) {
                        bulk_copy_g2s_hint(smem + pre * stage_sz + lane * kBlock,
                                           P.b_image + (static_cast<size_t>(n_blk) * P.k_stages + ks) * (2 * kBlock) + lane * kBlock,
                                           kBlock, &ctl->full[pre], weights_policy);
                    }
                }
            }
        }
        pdl_wait_prior_grids();
        if (lane == 0) TL(2);
        int it = 0;
        for (int w = blockIdx.x; w < total_items && !stop; w += gridDim.x) {
            const int tile = w / splits;
            const int ks0 = (w - tile * splits) * P.stages_per_split;
            const int ks1 = min(P.k_stages, ks0 + P.stages_per_split);
            const int m_blk = tile % P.m_blocks;
            const int n_blk = tile / P.m_blocks;
            for (int ks = ks0; ks < ks1; ++ks, ++it) {
                int bad = 0;
                if (lane == 0) {
                    if (*abort_flag) {
                        bad = 1;
                    } else if (it < pre) {
                        // barrier already armed, B half already on its way
                    } else if (wrapped && !mbar_wait_bounded(&ctl->empty[s], empty_phase)) {
                        record_error(kErrGemmEmptyBarrierTimeout);
                        *abort_flag = 1;
                        bad = 1;
                    } else {
                        mbar_expect_tx(&ctl->full[s], stage_sz);
                    }
                }
                bad = __shfl_sync(0xffffffffu, bad, 0);
                if (bad) {
                    stop = true;
                    break;
                }
                uint8_t* st = smem + s * stage_sz;
                if (kTiled) {
                    if (lane < 2 + pieces && (lane >= 2 || it >= pre)) {
                        const uint8_t* src =
                            lane < 2 ? P.b_image + (static_cast<size_t>(n_blk) * P.k_stages + ks) * (2 * kBlock) + lane * kBlock
                                     : P.a_image + (static_cast<size_t>(m_blk) * P.k_stages + ks) * (pieces * kBlock) +
                                           (lane - 2) * kBlock;
                        if (lane < 2) bulk_copy_g2s_hint(st + lane * kBlock, src, kBlock, &ctl->full[s], weights_policy);
                        else bulk_copy_g2s(st + lane * kBlock, src, kBlock, &ctl->full[s]);
                    }
                } else if (lane == 0) {
                    tc::tma_load_2d(st, &P.map_b, ks * kBKBytes, n_blk * kBN, &ctl->full[s]);
                } else if (lane == 1) {
                    bulk_copy_g2s(st + off_sfb,
                                  P.sfb + static_cast<size_t>(n_blk) * sf_row_stride + static_cast<size_t>(ks) * kSfSlab,
                                  kSfSlab, &ctl->full[s]);
                } else if (lane < 2 + 2 * pieces) {
                    const int p = (lane - 2) >> 1;
                    const int a_row_tile = p * (P.a_piece_rows >> 7) + m_blk;
                    if ((lane & 1) == 0) {
                        tc::tma_load_2d(st + off_a + p * kTile, &P.map_a, ks * kBKBytes, a_row_tile * kBM, &ctl->full[s]);
                    } else {
                        bulk_copy_g2s(st + off_sfa + p * kSfSlab,
                                      P.sfa + static_cast<size_t>(a_row_tile) * sf_row_stride +
                                          static_cast<size_t>(ks) * kSfSlab,
                                      kSfSlab, &ctl->full[s]);
                    }
                }
                if (++s == nstages) {
                    s = 0;
                    empty_phase ^= wrapped ? 1u : 0u;
                    wrapped = true;
                }
            }
            if (lane == 0 && w == blockIdx.x) TL(3);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = tc::make_idesc_mxf4nvf4(kBN);
            // descriptor words: (stage base >> 4) + compile-time offsets; see tcgen05.cuh
            const uint32_t stage16 = static_cast<uint32_t>(stage_sz) >> 4;
            const uint32_t off_a16 = static_cast<uint32_t>(off_a) >> 4;
            const uint32_t off_sfb16 = static_cast<uint32_t>(off_sfb) >> 4;
            const uint32_t off_sfa16 = static_cast<uint32_t>(off_sfa) >> 4;
            const uint32_t base16 = smem_u32(smem) >> 4;
            const uint32_t t_sfa = tmem_base + kSfaCol;
            const uint32_t t_sfb = tmem_base + kSfbCol;
            int s = 0;
            uint32_t full_phase = 0;
            uint32_t lo0 = base16;                 // descriptor word of the current stage's first byte
            int tile_iter = 0;
            for (int w = blockIdx.x; w < total_items && !*abort_flag; w += gridDim.x, ++tile_iter) {
                const int ks0 = (w % splits) * P.stages_per_split;
                const int ks1 = min(P.k_stages, ks0 + P.stages_per_split);
                const int buf = tile_iter % kAccBufs;
                const int use = tile_iter / kAccBufs;
                if (use >= 1 && !mbar_wait_bounded(&ctl->acc_empty[buf], (use - 1) & 1)) {
                    record_error(kErrGemmEpilogueBarrierTimeout);
                    *abort_flag = 1;
                    break;
                }
                tc::fence_after_thread_sync();
                const uint32_t tmem_acc = tmem_base + buf * 128;
                uint32_t accumulate = 0;           // the first MMA of the item overwrites the accumulator
                for (int ks = ks0; ks < ks1; ++ks) {
                    if (!mbar_wait_bounded(&ctl->full[s], full_phase)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    if (tile_iter == 0 && ks == ks0) TL(4);
                    // B scales of K atom a sit in kSubTiles * 4 consecutive columns (4 per 128 rows)
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
#pragma unroll
                        for (int h = 0; h < kSubTiles; ++h) {
                            tc::cp_sf_32x128b(t_sfb + 4 * (kSubTiles * a + h),
                                              tc::desc_from_words(lo0 + off_sfb16 + ((h * kSfSlab + a * 512) >> 4),
                                                                  tc::kDescHiSfAtom));
                        }
                    }
                    uint32_t lo_a = lo0 + off_a16;         // piece p's code tile
                    uint32_t lo_sfa = lo0 + off_sfa16;     // piece p's scale slab
                    uint32_t t_sfa_p = t_sfa;
                    for (int p = 0; p < pieces; ++p) {
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            tc::cp_sf_32x128b(t_sfa_p + 4 * a,
                                              tc::desc_from_words(lo_sfa + ((a * 512) >> 4), tc::kDescHiSfAtom));
                        }
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            tc::mma_mxf4nvf4(tmem_acc, tc::desc_from_words(lo_a + ((a * 32) >> 4), tc::kDescHiKmajorSw128),
                                             tc::desc_from_words(lo0 + ((a * 32) >> 4), tc::kDescHiKmajorSw128), idesc,
                                             t_sfa_p + 4 * a, t_sfb + 4 * kSubTiles * a, accumulate);
                            accumulate = 1;
                        }
                        lo_a += kTile >> 4;
                        lo_sfa += kSfSlab >> 4;
                        t_sfa_p += 16;
                    }
                    tc::commit(&ctl->empty[s]);   // stage s may be refilled once these MMAs have read it
                    if (++s == nstages) {
                        s = 0;
                        full_phase ^= 1;
                        lo0 = base16;
                    } else {
                        lo0 += stage16;
                    }
                }
                tc::commit(&ctl->acc_full[buf]);  // accumulator complete
                if (tile_iter == 0) TL(5);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
        const int q = warp & 3;                       // tensor-memory lane quarter this warp may read
        const int row = q * 32 + lane;                // row of the tile this thread owns
        const int grp = (warp - 2) >> 2;              // epilogue group 0 (warps 2..5) or 1 (warps 6..9)
        const int etid = (threadIdx.x - 64) & 127;    // 0..127 inside the group
        const bool issuer = (etid == 0);              // the group's first thread issues its TMA stores
        const bool at_work = grp == 0 || two_groups;
        const int n_heads_q = P.q_dim >> 8;
        int tile_iter = 0;
        uint32_t nstore = 0;                          // staged boxes so far (buffer = nstore & 1)
        for (int w = blockIdx.x; at_work && w < total_items && !*abort_flag; w += gridDim.x, ++tile_iter) {
            const int tile = w / splits;
            const int m_blk = tile % P.m_blocks;
            const int n_blk = tile / P.m_blocks;
            const int buf = tile_iter % kAccBufs;
            if (!mbar_wait_bounded(&ctl->acc_full[buf], (tile_iter / kAccBufs) & 1)) {
                record_error(kErrGemmMmaBarrierTimeout);
                *abort_flag = 1;
                break;
            }
            tc::fence_after_thread_sync();
            if (issuer && tile_iter == 0) TL(6);
            const int m = m_blk * kBM + row;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 128;
            const float rs = (P.row_scale != nullptr && m < P.M) ? P.alpha * __ldg(P.row_scale + m) : P.alpha;

            if (splits > 1) {
                // ---- split K: every CTA of the tile parks its partial sums, waits until all of them
                // have, then finishes its own slice of the tile's rows (sum in split order, epilogue
                // arithmetic, plain vector stores).  All CTAs of the launch are resident (grid <= SMs,
                // one CTA per SM) and nobody waits before parking, so the wait cannot deadlock; it is
                // bounded all the same.
                const int rows_valid = min(kBM, P.M - m_blk * kBM);
                float4* scratch4 = reinterpret_cast<float4*>(P.scratch);
                if (q * 32 < rows_valid) {     // whole warps only: the tensor-memory load is warp-collective
                    float4* dst = scratch4 + static_cast<size_t>(w) * kItemFloat4 + row;
                    // four tensor-memory loads in flight per wait: the parking pass is on every split launch's
                    // critical path (all CTAs of the tile wait for the slowest one to finish it)
#pragma unroll 1
                    for (int c4 = 0; c4 < kBN / 128; ++c4) {
                        uint32_t r[4][32];
#pragma unroll
                        for (int c = 0; c < 4; ++c) tc::tmem_ld_32x32b_x32(taddr + (c4 * 4 + c) * 32, r[c]);
                        tc::tmem_ld_wait();
                        if (row < rows_valid) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
#pragma unroll
                                for (int g = 0; g < 8; ++g) {
                                    dst[((c4 * 4 + c) * 8 + g) * 128] =
                                        make_float4(__uint_as_float(r[c][4 * g]), __uint_as_float(r[c][4 * g + 1]),
                                                    __uint_as_float(r[c][4 * g + 2]), __uint_as_float(r[c][4 * g + 3]));
                                }
                            }
                        }
                    }
                }
                tc::fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                __threadfence();
                epilogue_barrier();
                if (issuer) {
                    atomicAdd(P.counters + tile, 1u);
                    if (tile_iter == 0) TL(7);
                    const long long t0 = clock64();
                    while (true) {
                        unsigned int seen;
                        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(P.counters + tile) : "memory");
                        if (seen >= static_cast<unsigned int>(splits)) break;
                        if (clock64() - t0 > 2000000000LL) {
                            record_error(kErrGemmSplitTimeout);
                            *abort_flag = 1;
                            break;
                        }
                    }
                }
                epilogue_barrier();
                if (*abort_flag) break;
                __threadfence();
                if (issuer && tile_iter == 0) TL(8);
                const int split = w - tile * splits;
                const int per = (rows_valid + splits - 1) / splits;
                const int r0 = split * per;
                const int nrows = max(0, min(rows_valid, r0 + per) - r0);
                const float4* part = scratch4 + static_cast<size_t>(tile) * splits * kItemFloat4;
                auto sum32 = [&](int r, int col, float* v) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = 0.0f;
#pragma unroll 2
                    for (int sp = 0; sp < splits; ++sp) {
                        const float4* src = part + static_cast<size_t>(sp) * kItemFloat4 + (col >> 2) * 128 + r;
#pragma unroll
                        for (int g = 0; g < 8; ++g) {
                            const float4 t = __ldcg(src + g * 128);
                            v[4 * g] += t.x; v[4 * g + 1] += t.y; v[4 * g + 2] += t.z; v[4 * g + 3] += t.w;
                        }
                    }
                };
                if (P.epilogue == kEpiPlain && nrows * (kBN / 32) <= 32 &&
                    !(kTiled && P.activation == TPB200_ACT_GEGLU)) {
                    // Few rows per CTA (the 50-token launches cut 8 or 16 ways): units of 8 columns instead of 32
                    // put all 128 threads to work and leave each with 2 loads per split instead of 8 -- the pass
                    // is a chain of L2 round trips, and this is the tail of a latency-bound launch.
                    const int units = nrows * (kBN / 8);
                    for (int u = etid; u < units; u += 128) {
                        const int r = r0 + u % nrows;
                        const int c8 = u / nrows;
                        const int n = n_blk * kBN + c8 * 8;
                        if (n >= P.N) continue;
                        const int mm = m_blk * kBM + r;
                        const float rs_mm = P.row_scale != nullptr ? P.alpha * __ldg(P.row_scale + mm) : P.alpha;
                        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        const float4* src = part + (c8 * 2) * 128 + r;
#pragma unroll 4
                        for (int sp = 0; sp < splits; ++sp) {
                            const float4 t0 = __ldcg(src + static_cast<size_t>(sp) * kItemFloat4);
                            const float4 t1 = __ldcg(src + static_cast<size_t>(sp) * kItemFloat4 + 128);
                            v[0] += t0.x; v[1] += t0.y; v[2] += t0.z; v[3] += t0.w;
                            v[4] += t1.x; v[5] += t1.y; v[6] += t1.z; v[7] += t1.w;
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            v[i] *= rs_mm;
                            if (P.bias != nullptr && n + i < P.N) v[i] += __ldg(P.bias + n + i);
                            if (P.activation == TPB200_ACT_GELU) v[i] = gelu_tanh_fast(v[i]);
                            else if (P.activation == TPB200_ACT_SILU) v[i] = silu_fast(v[i]);
                        }
                        if (P.out_dtype == TPB200_BF16) {
                            uint32_t pk[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                                pk[i] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(P.out) + static_cast<size_t>(mm) * P.ldo + n;
                            if (n + 8 <= P.N) {
                                *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            } else {
                                for (int i = 0; n + i < P.N; ++i) dst[i] = __float2bfloat16_rn(v[i]);
                            }
                        } else {
                            float* dst = static_cast<float*>(P.out) + static_cast<size_t>(mm) * P.ldo + n;
                            if (n + 8 <= P.N) {
                                reinterpret_cast<float4*>(dst)[0] = make_float4(v[0], v[1], v[2], v[3]);
                                reinterpret_cast<float4*>(dst)[1] = make_float4(v[4], v[5], v[6], v[7]);
                            } else {
                                for (int i = 0; n + i < P.N; ++i) dst[i] = v[i];
                            }
                        }
                    }
                } else if (P.epilogue == kEpiPlain) {
                    const bool geglu = kTiled && P.activation == TPB200_ACT_GEGLU;
                    const int out_cols = geglu ? 128 : kBN;          // output columns of this tile
                    const int n_out = geglu ? P.N >> 1 : P.N;
                    const int units = nrows * (out_cols / 32);
                    for (int u = etid; u < units; u += 128) {
                        const int r = r0 + u % nrows;
                        const int c = u / nrows;
                        const int n = n_blk * out_cols + c * 32;
                        if (n >= n_out) continue;
                        const int mm = m_blk * kBM + r;
                        const float rs_mm = P.row_scale != nullptr ? P.alpha * __ldg(P.row_scale + mm) : P.alpha;
                        float v[32];
                        sum32(r, c * 32, v);
                        if (geglu) {
                            float up[32];
                            sum32(r, 128 + c * 32, up);
                            finish_geglu32(v, up, rs_mm);
                        } else {
                            finish_plain32(v, rs_mm, P.bias, n, P.N, P.activation);
                        }
                        if (P.out_dtype == TPB200_BF16) {
                            uint32_t pk[16];
                            pack_bf16x32(v, pk);
                            uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(P.out) +
                                                                  static_cast<size_t>(mm) * P.ldo + n);
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (n + 8 * g < n_out) dst[g] = make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
                            }
                        } else {
                            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(P.out) +
                                                                    static_cast<size_t>(mm) * P.ldo + n);
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                if (n + 4 * g < n_out) dst[g] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                            }
                        }
                    }
                } else {
                    const int units = nrows * (kBN / 64);
                    for (int u = etid; u < units; u += 128) {
                        const int r = r0 + u % nrows;
                        const int cu = u / nrows;                  // (128-column half, 32-column chunk)
                        const int sub = cu >> 1, c = cu & 1;
                        const int n128 = n_blk * kSubTiles + sub;
                        const int head = n128 >> 1;
                        const int i = (n128 & 1) * 64 + c * 32;    // head offset of the first lo column
                        const bool is_v = head == n_heads_q + 1;
                        const int mm = m_blk * kBM + r;
                        float lo[32], hi[32];
                        sum32(r, sub * 128 + c * 32, lo);
                        sum32(r, sub * 128 + 64 + c * 32, hi);
                        const int pos = __ldg(P.positions + mm);
                        uint32_t olo[16], ohi[16];
                        rope_pair32(lo, hi, P.row_scale != nullptr ? P.alpha * __ldg(P.row_scale + mm) : P.alpha,
                                    P.rope_cos + static_cast<size_t>(pos) * 128 + i,
                                    P.rope_sin + static_cast<size_t>(pos) * 128 + i, is_v, olo, ohi);
                        __nv_bfloat16* base = head < n_heads_q
                                                  ? static_cast<__nv_bfloat16*>(P.out) + static_cast<size_t>(mm) * P.ldo + head * 256
                                                  : (is_v ? P.v_rows : P.k_rows) + static_cast<size_t>(mm) * 256;
                        uint4* dlo = reinterpret_cast<uint4*>(base + i);
                        uint4* dhi = reinterpret_cast<uint4*>(base + i + 128);
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            dlo[g] = make_uint4(olo[4 * g], olo[4 * g + 1], olo[4 * g + 2], olo[4 * g + 3]);
                            dhi[g] = make_uint4(ohi[4 * g], ohi[4 * g + 1], ohi[4 * g + 2], ohi[4 * g + 3]);
                        }
                    }
                }
                // the last CTA to leave the tile puts both counters back to zero for the next launch
                epilogue_barrier();
                if (issuer && tile_iter == 0) TL(9);
                if (issuer) {
                    const unsigned int t = atomicAdd(P.counters + kCounterSlots + tile, 1u);
                    if (t == static_cast<unsigned int>(splits - 1)) {
                        P.counters[tile] = 0;
                        P.counters[kCounterSlots + tile] = 0;
                    }
                }
                continue;
            }

            if (P.epilogue == kEpiPlain) {
                // boxes of 128 bytes per row: 64 bf16 or 32 fp32 columns
                // gated GELU (tiled form): tile columns [0, 128) are gate outputs, [128, 256) the matching
                // up outputs; the tile yields 128 output columns
                const bool geglu = kTiled && P.activation == TPB200_ACT_GEGLU;
                const int out_cols = geglu ? 128 : kBN;
                const int n_out = geglu ? P.N >> 1 : P.N;
                const int cols_per_box = P.out_dtype == TPB200_BF16 ? 64 : 32;
                const int nboxes = out_cols / cols_per_box;
                uint8_t* ob = out_stage + grp * kOutBuf;      // one staging buffer per group
                float* bias_s = ctl->bias_s[grp];
                const bool has_bias = P.bias != nullptr;
                if (P.out_dtype == TPB200_BF16 && !geglu && nboxes == 4) {
                    // bf16, 256-column tile: the group's two boxes (columns [64 g, 64 g + 64) and 128 further on)
                    // are converted straight out of tensor memory into 64 packed registers, and the accumulator
                    // is handed back to the MMA thread BEFORE anything is staged or stored: the single
                    // accumulator is free again after four loads instead of after the whole epilogue.
                    if (has_bias) {
                        const int nb = n_blk * kBN + (etid >> 6) * 128 + grp * 64 + (etid & 63);
                        bias_s[etid] = nb < P.N ? __ldg(P.bias + nb) : 0.0f;
                    }
                    epilogue_group_barrier(grp);
                    uint32_t pk[4][16];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t raw[32];
                        tc::tmem_ld_32x32b_x32(taddr + (c >> 1) * 128 + grp * 64 + (c & 1) * 32, raw);
                        tc::tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                        finish_plain32_staged(v, rs, bias_s + c * 32, has_bias, P.activation);
                        pack_bf16x32(v, pk[c]);
                    }
                    tc::fence_before_thread_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
#pragma unroll
                    for (int b2 = 0; b2 < 2; ++b2) {
                        const int n0 = n_blk * kBN + b2 * 128 + grp * 64;
                        if (issuer) bulk_wait_group_read<0>();    // the group's previous store has read the buffer
                        epilogue_group_barrier(grp);
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                *reinterpret_cast<uint4*>(staged_chunk(ob, row, c * 4 + g)) =
                                    make_uint4(pk[b2 * 2 + c][4 * g], pk[b2 * 2 + c][4 * g + 1], pk[b2 * 2 + c][4 * g + 2],
                                               pk[b2 * 2 + c][4 * g + 3]);
                            }
                        }
                        fence_proxy_async_smem();
                        epilogue_group_barrier(grp);
                        if (issuer) {
                            if (n0 < n_out) tma_store_2d(&P.map_out, ob, n0, m_blk * kBM);
                            bulk_commit_group();
                        }
                    }
                    continue;
                }
                if (P.out_dtype == TPB200_BF16 && geglu) {
                    // Gated GELU, bf16: the group's 64 gate columns and their 64 up columns leave tensor memory as
                    // bf16 pairs (the module rounds both projections to bf16 before the activation anyway), the
                    // accumulator goes back to the MMA thread, and only then comes the GELU arithmetic.
                    uint32_t gpk[2][16], upk[2][16];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        uint32_t raw[32];
                        tc::tmem_ld_32x32b_x32(taddr + (c >> 1) * 128 + grp * 64 + (c & 1) * 32, raw);
                        tc::tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]) * rs;
                        pack_bf16x32(v, c < 2 ? gpk[c & 1] : upk[c & 1]);
                    }
                    tc::fence_before_thread_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                    const int n0 = n_blk * 128 + grp * 64;
                    if (issuer) bulk_wait_group_read<0>();    // the group's previous store has read the buffer
                    epilogue_group_barrier(grp);
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        uint32_t o[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float2 gb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gpk[c][i]));
                            const float2 ub = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&upk[c][i]));
                            const float a0 = __bfloat162float(__float2bfloat16_rn(gelu_tanh_fast(gb.x))) * ub.x;
                            const float a1 = __bfloat162float(__float2bfloat16_rn(gelu_tanh_fast(gb.y))) * ub.y;
                            const __nv_bfloat162 r2 = __floats2bfloat162_rn(a0, a1);
                            o[i] = *reinterpret_cast<const uint32_t*>(&r2);
                        }
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            *reinterpret_cast<uint4*>(staged_chunk(ob, row, c * 4 + g)) =
                                make_uint4(o[4 * g], o[4 * g + 1], o[4 * g + 2], o[4 * g + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    epilogue_group_barrier(grp);
                    if (issuer) {
                        if (n0 < n_out) tma_store_2d(&P.map_out, ob, n0, m_blk * kBM);
                        bulk_commit_group();
                    }
                    continue;
                }
#pragma unroll 1
                for (int bx = grp; bx < nboxes; bx += 2) {
                    const int n0 = n_blk * out_cols + bx * cols_per_box;
                    if (has_bias && !geglu && etid < cols_per_box) {
                        bias_s[etid] = n0 + etid < P.N ? __ldg(P.bias + n0 + etid) : 0.0f;
                    }
                    if (issuer) bulk_wait_group_read<0>();    // the group's previous store has read the buffer
                    epilogue_group_barrier(grp);
#pragma unroll 1
                    for (int c = 0; c < cols_per_box / 32; ++c) {
                        uint32_t raw[32];
                        tc::tmem_ld_32x32b_x32(taddr + bx * cols_per_box + c * 32, raw);
                        tc::tmem_ld_wait();
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
                        if (geglu) {
                            tc::tmem_ld_32x32b_x32(taddr + 128 + bx * cols_per_box + c * 32, raw);
                            tc::tmem_ld_wait();
                            float up[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) up[i] = __uint_as_float(raw[i]);
                            finish_geglu32(v, up, rs);
                        } else {
                            finish_plain32_staged(v, rs, bias_s + c * 32, has_bias, P.activation);
                        }
                        if (P.out_dtype == TPB200_BF16) {
                            uint32_t pk[16];
                            pack_bf16x32(v, pk);
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                *reinterpret_cast<uint4*>(staged_chunk(ob, row, c * 4 + g)) =
                                    make_uint4(pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
                            }
                        } else {
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                *reinterpret_cast<float4*>(staged_chunk(ob, row, g)) =
                                    make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                            }
                        }
                    }
                    if (bx + 2 >= nboxes) {
                        // everything this warp needs from the accumulator is in registers / shared memory
                        tc::fence_before_thread_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                    }
                    fence_proxy_async_smem();
                    epilogue_group_barrier(grp);
                    if (issuer) {
                        if (n0 < n_out) tma_store_2d(&P.map_out, ob, n0, m_blk * kBM);
                        bulk_commit_group();
                    }
                }
            } else {
                // Fused QKV: tile columns [0,64) are head offsets i0..i0+63, columns [64,128) their
                // rotation partners i + 128.  Two boxes of 64 columns per 128-column half: lo and hi.
                const int pos = (m < P.M) ? __ldg(P.positions + m) : 0;
                uint8_t* ob_lo = out_stage;
                uint8_t* ob_hi = out_stage + kOutBuf;
#pragma unroll 1
                for (int sub = 0; sub < kSubTiles; ++sub) {
                    const int n128 = n_blk * kSubTiles + sub;     // 128-row tile of the permuted weight
                    const int head = n128 >> 1;
                    const int i0 = (n128 & 1) * 64;
                    const bool is_v = head == n_heads_q + 1;
                    if (issuer) bulk_wait_group_read<0>();
                    epilogue_barrier();
#pragma unroll 1
                    for (int c = 0; c < 2; ++c) {
                        uint32_t rl[32], rh[32];
                        tc::tmem_ld_32x32b_x32(taddr + sub * 128 + c * 32, rl);
                        tc::tmem_ld_32x32b_x32(taddr + sub * 128 + 64 + c * 32, rh);
                        tc::tmem_ld_wait();
                        if (c == 1 && sub == kSubTiles - 1) {
                            tc::fence_before_thread_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                        }
                        float lo[32], hi[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            lo[i] = __uint_as_float(rl[i]);
                            hi[i] = __uint_as_float(rh[i]);
                        }
                        const int i = i0 + c * 32;   // head offset of lo[0]
                        uint32_t olo[16], ohi[16];
                        rope_pair32(lo, hi, rs, P.rope_cos + static_cast<size_t>(pos) * 128 + i,
                                    P.rope_sin + static_cast<size_t>(pos) * 128 + i, is_v, olo, ohi);
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            *reinterpret_cast<uint4*>(staged_chunk(ob_lo, row, c * 4 + g)) =
                                make_uint4(olo[4 * g], olo[4 * g + 1], olo[4 * g + 2], olo[4 * g + 3]);
                            *reinterpret_cast<uint4*>(staged_chunk(ob_hi, row, c * 4 + g)) =
                                make_uint4(ohi[4 * g], ohi[4 * g + 1], ohi[4 * g + 2], ohi[4 * g + 3]);
                        }
                    }
                    fence_proxy_async_smem();
                    epilogue_barrier();
                    if (issuer) {
                        const CUtensorMap* map = head < n_heads_q ? &P.map_out : (is_v ? &P.map_v : &P.map_k);
                        const int x0 = head < n_heads_q ? head * 256 + i0 : i0;
                        tma_store_2d(map, ob_lo, x0, m_blk * kBM);
                        tma_store_2d(map, ob_hi, x0 + 128, m_blk * kBM);
                        bulk_commit_group();
                    }
                    nstore += 2;
                }
            }
        }
        if (issuer) bulk_wait_group_all();   // every output tile has landed before the CTA goes away
        if (issuer) TL(10);
    }

    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// Measurement utility: the e2m1 block-scaled MMA rate of this GPU with nothing else in the way.  One CTA per
// SM issues `mmas` MMAs of 128 x 256 x 64 back to back on operands that already sit in shared memory (no
// loads, no epilogue), so FLOPs / time is the tensor pipe's own pace at the clocks the run gets.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64, 1) fp4_mma_rate_kernel(int mmas) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // [B 256 rows x 128 B][A 128 rows x 128 B][B scale slabs 2 x 2 KB][A scale slab 2 KB][barrier, tmem address]
    uint8_t* sB = smem;
    uint8_t* sA = sB + 2 * kTile;
    uint8_t* sSfb = sA + kTile;
    uint8_t* sSfa = sSfb + 2 * kSfSlab;
    uint64_t* bar = reinterpret_cast<uint64_t*>(sSfa + kSfSlab);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    for (int i = threadIdx.x; i < 3 * kTile / 4; i += 64) reinterpret_cast<uint32_t*>(smem)[i] = 0x2A2A2A2Au;   // codes 1.0 / -1.0
    for (int i = threadIdx.x; i < 3 * kSfSlab / 4; i += 64) reinterpret_cast<uint32_t*>(sSfb)[i] = 0x38383838u; // UE4M3 1.0
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        fence_mbar_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x >= 32) {
        __syncwarp();
        tc::tmem_alloc(tmem_slot, kTmemCols);
        tc::tmem_relinquish();
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = tc::make_idesc_mxf4nvf4(256);
        const uint32_t b16 = smem_u32(sB) >> 4, a16 = smem_u32(sA) >> 4;
        const uint32_t sfb16 = smem_u32(sSfb) >> 4, sfa16 = smem_u32(sSfa) >> 4;
        const uint32_t t_sfb = tmem_base + kSfbCol, t_sfa = tmem_base + kSfaCol;
        for (int a = 0; a < 4; ++a) {
            for (int h = 0; h < 2; ++h) {
                tc::cp_sf_32x128b(t_sfb + 4 * (2 * a + h), tc::desc_from_words(sfb16 + ((h * kSfSlab + a * 512) >> 4), tc::kDescHiSfAtom));
            }
            tc::cp_sf_32x128b(t_sfa + 4 * a, tc::desc_from_words(sfa16 + ((a * 512) >> 4), tc::kDescHiSfAtom));
        }
        uint32_t accumulate = 0;
        for (int i = 0; i < mmas; ++i) {
            const int a = i & 3;
            tc::mma_mxf4nvf4(tmem_base, tc::desc_from_words(a16 + ((a * 32) >> 4), tc::kDescHiKmajorSw128),
                             tc::desc_from_words(b16 + ((a * 32) >> 4), tc::kDescHiKmajorSw128), idesc, t_sfa + 4 * a,
                             t_sfb + 8 * a, accumulate);
            accumulate = 1;
        }
        tc::commit(bar);
        if (!mbar_wait_bounded(bar, 0)) record_error(kErrGemmMmaBarrierTimeout);
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    if (threadIdx.x >= 32) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// Weight preparation for the tiled form: row-major codes [N, pitch] + atom-layout scales -> B image.
// Block (n_blk, ks) of 36 KB: 256 rows x 128 B with 16-byte chunk c of row r stored at c ^ (r & 7),
// then the 2 KB scale slabs of rows [0, 128) and [128, 256).  Rows >= N and K beyond the matrix are
// zero codes with zero scales.  One thread per 16-byte chunk of the image.
// ------------------------------------------------------------------------------------------
__global__ void tile_weights_kernel(const uint8_t* __restrict__ packed, int pitch, const uint8_t* __restrict__ sf,
                                    uint8_t* __restrict__ image, int N, int K, int k_stages, long long chunks) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= chunks) return;
    constexpr int kChunksPerBlock = 2 * kBlock / 16;
    const long long blk = t / kChunksPerBlock;
    const int ci = static_cast<int>(t % kChunksPerBlock);
    const int n_blk = static_cast<int>(blk / k_stages);
    const int ks = static_cast<int>(blk % k_stages);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (ci < 2 * kTile / 16) {
        const int r = ci >> 3;                 // row of the 256-row block
        const int c = (ci & 7) ^ (r & 7);      // source chunk that lands in this slot
        const int n = n_blk * 256 + r;
        const int byte0 = ks * 128 + c * 16;
        if (n < N && byte0 < K / 2) {
            v = *reinterpret_cast<const uint4*>(packed + static_cast<size_t>(n) * pitch + byte0);
            // a chunk that straddles K / 2 (K % 32 != 0) keeps only its valid bytes
            const int valid = K / 2 - byte0;
            if (valid < 16) {
                uint32_t w[4] = {v.x, v.y, v.z, v.w};
                for (int i = 0; i < 4; ++i) {
                    const int rem = valid - 4 * i;
                    if (rem <= 0) w[i] = 0;
                    else if (rem < 4) w[i] &= (1u << (8 * rem)) - 1u;
                }
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    } else {
        const int si = ci - 2 * kTile / 16;    // 16-byte chunk of the two scale slabs
        const int h = si / (kSfSlab / 16);
        const int off = (si % (kSfSlab / 16)) * 16;
        const int row_tile = n_blk * 2 + h;
        if (row_tile * 128 < N) {
            v = *reinterpret_cast<const uint4*>(sf + (static_cast<size_t>(row_tile) * k_stages + ks) * kSfSlab + off);
        }
    }
    *reinterpret_cast<uint4*>(image + static_cast<size_t>(t) * 16) = v;
}

// ------------------------------------------------------------------------------------------
// Activation quantiser: x [M, K] -> e2m1 codes [M, pitch] + UE4M3 scales in the atom layout.
// One thread per 16-element block over the PADDED scale domain, so padding scales are zeroed.
// Codes follow the reference's simulation quantiser
// (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:88-173 with use_mse_search=False):
//   sf = max(blockmax, 1e-12) / 6;  scaled = x / max(sf * 6, 1e-12) * 6, clamped to +-6;
//   nearest e2m1 magnitude (ties to the lower); a value that rounds to 0 is stored as +0.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e2m1_index(float a) {
    return (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
}

__global__ void nvfp4_quantize_act_kernel(const void* __restrict__ x, int x_dtype, int ldx, uint8_t* __restrict__ packed,
                                          int pitch, uint8_t* __restrict__ sf, int M, int K, int rows_pad,
                                          int kb_pad) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(rows_pad) * kb_pad) return;
    const int row = static_cast<int>(t / kb_pad);
    const int kb = static_cast<int>(t % kb_pad);
    const size_t sf_off = (static_cast<size_t>(row >> 7) * (kb_pad >> 2) + (kb >> 2)) * 512 + (row & 31) * 16 +
                          ((row >> 5) & 3) * 4 + (kb & 3);
    if (row >= M || kb * 16 >= K) {
        sf[sf_off] = 0;
        return;
    }
    float v[16];
    const size_t e0 = static_cast<size_t>(row) * ldx + static_cast<size_t>(kb) * 16;
    if (x_dtype == TPB200_F32) {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(x) + e0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float4 f = __ldg(p + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + e0);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            uint4 u = __ldg(p + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = x_dtype == TPB200_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&w[j]))
                                                 : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                v[8 * i + 2 * j] = f.x;
                v[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
    const float lim = 2688.0f;   // 448 * 6: keeps the block scale inside E4M3 (nvfp4_mlp.py:606-608)
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        v[i] = fminf(fmaxf(v[i], -lim), lim);
        amax = fmaxf(amax, fabsf(v[i]));
    }
    const float sfv = __fdiv_rn(fmaxf(amax, 1e-12f), 6.0f);
    const float denom = fmaxf(__fmul_rn(sfv, 6.0f), 1e-12f);
    sf[sf_off] = encode_e4m3(sfv);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        float s = __fmul_rn(__fdiv_rn(v[i], denom), 6.0f);
        s = fminf(fmaxf(s, -6.0f), 6.0f);
        const uint32_t idx = e2m1_index(fabsf(s));
        const uint32_t code = (s < 0.0f && idx != 0) ? (idx | 8u) : idx;
        if (i < 8) lo |= code << (4 * i);
        else hi |= code << (4 * (i - 8));
    }
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(row) * pitch + kb * 8) = make_uint2(lo, hi);
}

// ------------------------------------------------------------------------------------------
// Residual-piece activation quantiser: keeps (almost) the full precision of bf16 activations in
// e2m1 operands, so that weight-only semantics run on the block-scaled tensor-core path.
//   row pre-scale: x' = x * 2^e with max|x'| in [1024, 2048)   (row_scale[m] = 2^-e)
//   piece 0 quantises x', piece p quantises what pieces 0..p-1 left over, each per 16-block with
//   its own UE4M3 scale (rounded UP so that nothing clips):  x' ~= sum_p q_p * s_p.
// One CTA per row; piece p of row m goes to packed row p * piece_rows + m.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) nvfp4_quantize_pieces_kernel(const void* __restrict__ x, int x_dtype, int ldx,
                                                                    uint8_t* __restrict__ packed, int pitch,
                                                                    uint8_t* __restrict__ sf, float* __restrict__ row_scale,
                                                                    int M, int K, int pieces, int piece_rows,
                                                                    int kb_pad) {
    const int row = blockIdx.x;
    const int nblk = K >> 4;
    __shared__ float red[8];
    float amax = 0.0f;
    for (int kb = threadIdx.x; kb < nblk; kb += blockDim.x) {
        float r[16];
        load16_as_float(x, x_dtype, static_cast<size_t>(row) * ldx + kb * 16, r);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(r[i]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);        // amax = f * 2^ex, f in [0.5, 1)
        e = 11 - ex;              // amax * 2^e in [1024, 2048)
    }
    const float pre = ldexpf(1.0f, e);
    if (threadIdx.x == 0) row_scale[row] = ldexpf(1.0f, -e);

    for (int kb = threadIdx.x; kb < kb_pad; kb += blockDim.x) {
        float r[16];
        const bool valid = kb < nblk;
        if (valid) {
            load16_as_float(x, x_dtype, static_cast<size_t>(row) * ldx + kb * 16, r);
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] *= pre;
        }
        for (int p = 0; p < pieces; ++p) {
            const int prow = p * piece_rows + row;
            const size_t sf_off = (static_cast<size_t>(prow >> 7) * (kb_pad >> 2) + (kb >> 2)) * 512 + (prow & 31) * 16 +
                                  ((prow >> 5) & 3) * 4 + (kb & 3);
            if (!valid) {
                sf[sf_off] = 0;
                continue;
            }
            uint32_t lo, hi;
            sf[sf_off] = quantize_block16_piece(r, lo, hi);
            *reinterpret_cast<uint2*>(packed + static_cast<size_t>(prow) * pitch + kb * 8) = make_uint2(lo, hi);
        }
    }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn get_encode_fn() {
    static std::atomic<EncodeFn> cached{nullptr};
    EncodeFn fn = cached.load(std::memory_order_acquire);
    if (fn != nullptr) return fn;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || p == nullptr) {
        return nullptr;
    }
    fn = reinterpret_cast<EncodeFn>(p);
    cached.store(fn, std::memory_order_release);
    return fn;
}

}  // namespace

bool make_tensor_map_bytes_sw128(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                                 uint64_t pitch_bytes, uint32_t box_rows) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {128, box_rows};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// bf16 tensor of `rank` (2..5) dimensions, dims[0] contiguous, strides_bytes[i] = byte stride of dims[i + 1];
// box[0] <= 64 elements (one 128-byte swizzle row), elements past the end of a dimension read as zero.
bool make_tensor_map_bf16_nd_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                   const uint64_t* strides_bytes, const uint32_t* box) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr || rank < 2 || rank > 5) return false;
    cuuint64_t d[5], st[4];
    cuuint32_t b[5], es[5];
    for (int i = 0; i < rank; ++i) {
        d[i] = dims[i];
        b[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) st[i] = strides_bytes[i];
    }
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base), d, st, b, es,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Output matrix [rows, cols] of bf16 / fp32 elements, box = 128 rows x 128 bytes, 128-byte swizzle.
bool make_tensor_map_out_sw128(CUtensorMap* map, void* base, int dtype, uint64_t cols, uint64_t rows,
                               uint64_t pitch_bytes) {
    EncodeFn fn = get_encode_fn();
    if (fn == nullptr) return false;
    const bool bf = dtype == TPB200_BF16;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {bf ? 64u : 32u, 128u};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, bf ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box,
              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int device_error_nvfp4_gemm(int clear) { return read_device_error(clear); }

// Split-K plan.  A launch with fewer tiles than SMs leaves SMs idle and makes each busy one walk the
// whole K range; splitting K over `splits` CTAs per tile trades that for one pass of the partial sums
// through L2.  The cost model (microseconds, fitted to B200 timings of this kernel) only has to rank
// the candidates.
constexpr size_t kCounterBytes = 16384;            // 4096 tile counters in front of the partial sums
struct SplitPlan { int splits; int stages_per_split; size_t bytes; };

SplitPlan plan_splits(int tiles, int k_stages, int pieces, bool tiled, int sms, size_t workspace_bytes, int rows) {
    SplitPlan best{1, k_stages, 0};
    if (2 * tiles > sms || tiles > kCounterSlots || k_stages < 2) return best;
    const size_t item_bytes = static_cast<size_t>(128) * tile_n(tiled) * 4;   // one partial accumulator
    // Device timestamps of this kernel (three pieces, tiled): a stage takes 1.4 us (two stages of 90 KB in
    // flight per SM); a split launch adds parking the sums (1.8 us for 50 valid rows, 3.4 for 128), the wait for
    // the slowest partner (1-1.5 us) and the slice pass (1.7 / 4.4 us) where an unsplit tile has a 2 us epilogue.
    const float t_stage = stage_bytes(pieces, tiled) / 1024.0f / (tiled ? 64.0f : 70.0f);
    const float t_split = 1.0f + 0.05f * static_cast<float>(std::min(rows, 128));
    float best_cost = k_stages * t_stage;
    for (int s = 2; s <= std::min(k_stages, sms / tiles); ++s) {    // one wave: every CTA is resident
        const int sps = (k_stages + s - 1) / s;
        const int s_eff = (k_stages + sps - 1) / sps;
        const size_t bytes = kCounterBytes + static_cast<size_t>(tiles) * s_eff * item_bytes;
        if (bytes > workspace_bytes) continue;
        const float c = sps * t_stage + t_split;
        if (c < best_cost * 0.95f) {
            best_cost = c;
            best = SplitPlan{s_eff, sps, bytes};
        }
    }
    return best;
}

}  // namespace tpb

extern "C" size_t tpb200_nvfp4_sf_bytes(int rows, int K) {
    if (rows < 1 || K < 16) return 0;
    const size_t row_tiles = (static_cast<size_t>(rows) + 127) / 128;
    const size_t k_stages = (static_cast<size_t>(K) + 255) / 256;
    return row_tiles * k_stages * tpb::kSfSlab;
}

extern "C" int tpb200_nvfp4_quantize_act(const void* x, int x_dtype, int ldx, void* packed, int packed_pitch,
                                         void* sf_swizzled, int M, int K, tpb200_stream_t stream) {
    TPB_REQUIRE(x && packed && sf_swizzled, TPB200_ERR_NULL);
    TPB_REQUIRE(M >= 1 && K >= 16 && K % 16 == 0 && ldx >= K, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(x_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE(packed_pitch >= K / 2 && packed_pitch % 16 == 0, TPB200_ERR_ALIGN);
    TPB_REQUIRE(tpb_aligned16(x) && tpb_aligned16(packed) && tpb_aligned16(sf_swizzled), TPB200_ERR_ALIGN);
    TPB_REQUIRE((static_cast<long long>(ldx) * tpb_dtype_size(x_dtype)) % 16 == 0, TPB200_ERR_ALIGN);
    const int rows_pad = (M + 127) / 128 * 128;
    const int kb_pad = (K + 255) / 256 * 16;
    const long long total = static_cast<long long>(rows_pad) * kb_pad;
    const int threads = 256;
    tpb::nvfp4_quantize_act_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0,
                                     reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, ldx, static_cast<uint8_t*>(packed), packed_pitch, static_cast<uint8_t*>(sf_swizzled), M, K,
        rows_pad, kb_pad);
    return tpb_launch_status();
}

extern "C" int tpb200_nvfp4_quantize_act_pieces(const void* x, int x_dtype, int ldx, void* packed, int packed_pitch,
                                                void* sf_swizzled, float* row_scale, int M, int K, int pieces,
                                                int piece_rows, tpb200_stream_t stream) {
    TPB_REQUIRE(x && packed && sf_swizzled && row_scale, TPB200_ERR_NULL);
    TPB_REQUIRE(M >= 1 && K >= 16 && K % 16 == 0 && ldx >= K, TPB200_ERR_SHAPE);
    TPB_REQUIRE(pieces >= 1 && pieces <= 4 && piece_rows >= M, TPB200_ERR_SHAPE);
    TPB_REQUIRE(pieces == 1 || piece_rows % 16 == 0, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(x_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE(packed_pitch >= K / 2 && packed_pitch % 16 == 0, TPB200_ERR_ALIGN);
    TPB_REQUIRE(tpb_aligned16(x) && tpb_aligned16(packed) && tpb_aligned16(sf_swizzled), TPB200_ERR_ALIGN);
    TPB_REQUIRE((static_cast<long long>(ldx) * tpb_dtype_size(x_dtype)) % 16 == 0, TPB200_ERR_ALIGN);
    const int kb_pad = (K + 255) / 256 * 16;
    tpb::nvfp4_quantize_pieces_kernel<<<M, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        x, x_dtype, ldx, static_cast<uint8_t*>(packed), packed_pitch, static_cast<uint8_t*>(sf_swizzled), row_scale, M,
        K, pieces, piece_rows, kb_pad);
    return tpb_launch_status();
}

extern "C" size_t tpb200_nvfp4_tiled_a_bytes(int M, int K, int pieces) {
    if (M < 1 || K < 16 || pieces < 1 || pieces > 3) return 0;
    return static_cast<size_t>((M + 127) / 128) * ((K + 255) / 256) * pieces * tpb::kBlock;
}

extern "C" size_t tpb200_nvfp4_tiled_b_bytes(int N, int K) {
    if (N < 1 || K < 16) return 0;
    return static_cast<size_t>((N + 255) / 256) * ((K + 255) / 256) * 2 * tpb::kBlock;
}

extern "C" int tpb200_nvfp4_tile_weights(const void* packed, int pitch, const void* sf_swizzled, void* image, int N,
                                         int K, tpb200_stream_t stream) {
    TPB_REQUIRE(packed && sf_swizzled && image, TPB200_ERR_NULL);
    TPB_REQUIRE(N >= 1 && K >= 16 && K % 16 == 0, TPB200_ERR_SHAPE);
    TPB_REQUIRE(pitch >= K / 2 && pitch % 16 == 0 && tpb_aligned16(packed) && tpb_aligned16(sf_swizzled) &&
                    tpb_aligned16(image),
                TPB200_ERR_ALIGN);
    const int k_stages = (K + 255) / 256;
    const int n_blocks = (N + 255) / 256;
    const long long chunks = static_cast<long long>(n_blocks) * k_stages * (2 * tpb::kBlock / 16);
    tpb::tile_weights_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0,
                               reinterpret_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(packed), pitch, static_cast<const uint8_t*>(sf_swizzled),
        static_cast<uint8_t*>(image), N, K, k_stages, chunks);
    return tpb_launch_status();
}

extern "C" size_t tpb200_nvfp4_gemm_workspace_size(int M, int N, int K, int a_pieces, int layout) {
    if (M < 1 || N < 1 || K < 16) return 0;
    const bool tiled = layout == TPB200_OPERANDS_TILED;
    const int bn = tpb::tile_n(tiled);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return 0;
    }
    const int tiles = ((M + tpb::kBM - 1) / tpb::kBM) * ((N + bn - 1) / bn);
    return tpb::plan_splits(tiles, (K + 255) / 256, a_pieces <= 0 ? 1 : a_pieces, tiled, sms, ~size_t(0), M).bytes;
}

extern "C" int tpb200_nvfp4_gemm_ex(const tpb200_nvfp4_gemm_args* a, tpb200_stream_t stream) {
    TPB_REQUIRE(a != nullptr, TPB200_ERR_NULL);
    const int M = a->M, N = a->N, K = a->K;
    TPB_REQUIRE(a->layout == TPB200_OPERANDS_ROWMAJOR || a->layout == TPB200_OPERANDS_TILED, TPB200_ERR_ENUM);
    const bool tiled = a->layout == TPB200_OPERANDS_TILED;
    TPB_REQUIRE(a->a_packed && a->b_packed, TPB200_ERR_NULL);
    TPB_REQUIRE(M >= 1 && N >= 8 && N % 8 == 0 && K >= 16 && K % 16 == 0, TPB200_ERR_SHAPE);
    TPB_REQUIRE(a->activation >= TPB200_ACT_NONE && a->activation <= TPB200_ACT_GEGLU, TPB200_ERR_ENUM);
    const bool geglu = a->activation == TPB200_ACT_GEGLU;
    if (geglu) {
        TPB_REQUIRE(a->layout == TPB200_OPERANDS_TILED && a->qkv_q_out == nullptr && a->bias == nullptr, TPB200_ERR_ENUM);
        TPB_REQUIRE(N % 256 == 0, TPB200_ERR_SHAPE);
    }
    const int n_out = geglu ? N / 2 : N;
    const int pieces = a->a_pieces <= 0 ? 1 : a->a_pieces;
    TPB_REQUIRE(tpb_aligned16(a->a_packed) && tpb_aligned16(a->b_packed), TPB200_ERR_ALIGN);
    if (tiled) {
        TPB_REQUIRE(pieces <= 3, TPB200_ERR_SHAPE);
    } else {
        TPB_REQUIRE(a->a_sf && a->b_sf, TPB200_ERR_NULL);
        TPB_REQUIRE(a->a_pitch >= K / 2 && a->b_pitch >= K / 2 && a->a_pitch % 16 == 0 && a->b_pitch % 16 == 0,
                    TPB200_ERR_ALIGN);
        TPB_REQUIRE(tpb_aligned16(a->a_sf) && tpb_aligned16(a->b_sf), TPB200_ERR_ALIGN);
        TPB_REQUIRE(pieces <= 4, TPB200_ERR_SHAPE);
        TPB_REQUIRE(pieces == 1 || (a->a_piece_rows >= M && a->a_piece_rows % 128 == 0), TPB200_ERR_SHAPE);
    }
    const bool qkv = a->qkv_q_out != nullptr;
    if (qkv) {
        TPB_REQUIRE(a->qkv_k_rows && a->qkv_v_rows && a->qkv_positions && a->qkv_rope_cos && a->qkv_rope_sin,
                    TPB200_ERR_NULL);
        TPB_REQUIRE(a->qkv_q_dim >= 256 && a->qkv_q_dim % 256 == 0 && N == a->qkv_q_dim + 512 && a->qkv_ldq >= a->qkv_q_dim,
                    TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(a->qkv_q_out) && tpb_aligned16(a->qkv_k_rows) && tpb_aligned16(a->qkv_v_rows) &&
                        tpb_aligned16(a->qkv_rope_cos) && tpb_aligned16(a->qkv_rope_sin) && a->qkv_ldq % 8 == 0,
                    TPB200_ERR_ALIGN);
    } else {
        TPB_REQUIRE(a->out != nullptr, TPB200_ERR_NULL);
        TPB_REQUIRE(a->out_dtype == TPB200_BF16 || a->out_dtype == TPB200_F32, TPB200_ERR_ENUM);
        TPB_REQUIRE(a->ldo >= n_out, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(a->out) && (static_cast<long long>(a->ldo) * tpb_dtype_size(a->out_dtype)) % 16 == 0,
                    TPB200_ERR_ALIGN);
    }

    tpb::GemmParams P;
    const uint64_t a_rows = pieces == 1 ? static_cast<uint64_t>(M) : static_cast<uint64_t>(pieces) * a->a_piece_rows;
    if (!tiled &&
        (!tpb::make_tensor_map_bytes_sw128(&P.map_a, a->a_packed, static_cast<uint64_t>(K) / 2, a_rows, a->a_pitch,
                                           tpb::kBM) ||
         !tpb::make_tensor_map_bytes_sw128(&P.map_b, a->b_packed, static_cast<uint64_t>(K) / 2, N, a->b_pitch, 128))) {
        return TPB200_ERR_CUDA;
    }
    P.a_image = static_cast<const uint8_t*>(a->a_packed);
    P.b_image = static_cast<const uint8_t*>(a->b_packed);
    if (qkv) {
        if (!tpb::make_tensor_map_out_sw128(&P.map_out, a->qkv_q_out, TPB200_BF16, a->qkv_q_dim, M,
                                            static_cast<uint64_t>(a->qkv_ldq) * 2) ||
            !tpb::make_tensor_map_out_sw128(&P.map_k, a->qkv_k_rows, TPB200_BF16, 256, M, 512) ||
            !tpb::make_tensor_map_out_sw128(&P.map_v, a->qkv_v_rows, TPB200_BF16, 256, M, 512)) {
            return TPB200_ERR_CUDA;
        }
    } else {
        if (!tpb::make_tensor_map_out_sw128(&P.map_out, a->out, a->out_dtype, n_out, M,
                                            static_cast<uint64_t>(a->ldo) * tpb_dtype_size(a->out_dtype))) {
            return TPB200_ERR_CUDA;
        }
        P.map_k = P.map_out;
        P.map_v = P.map_out;
    }
    P.sfa = static_cast<const uint8_t*>(a->a_sf);
    P.sfb = static_cast<const uint8_t*>(a->b_sf);
    P.bias = a->bias;
    P.M = M; P.N = N; P.K = K;
    P.out_dtype = qkv ? TPB200_BF16 : a->out_dtype;
    P.activation = a->activation;
    P.alpha = a->alpha;
    P.k_stages = (K + 255) / 256;
    P.m_blocks = (M + tpb::kBM - 1) / tpb::kBM;
    P.n_blocks = (N + tpb::tile_n(tiled) - 1) / tpb::tile_n(tiled);
    P.a_pieces = pieces;
    P.a_piece_rows = pieces == 1 ? 0 : a->a_piece_rows;
    P.row_scale = a->a_row_scale;
    P.epilogue = qkv ? tpb::kEpiQkvRope : tpb::kEpiPlain;
    P.q_dim = a->qkv_q_dim;
    P.positions = a->qkv_positions;
    P.rope_cos = static_cast<const __nv_bfloat16*>(a->qkv_rope_cos);
    P.rope_sin = static_cast<const __nv_bfloat16*>(a->qkv_rope_sin);

    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    const size_t smem = tpb::num_stages(pieces, tiled) * tpb::stage_bytes(pieces, tiled) + 2 * tpb::kOutBuf +
                        sizeof(tpb::SharedControl) + 1024;
    static std::atomic<uint64_t> configured{0};
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(tpb::nvfp4_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024) != cudaSuccess ||
            cudaFuncSetAttribute(tpb::nvfp4_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    const int tiles = P.m_blocks * P.n_blocks;
    tpb::SplitPlan plan{1, P.k_stages, 0};
    if (a->workspace != nullptr) {
        TPB_REQUIRE(tpb_aligned16(a->workspace), TPB200_ERR_ALIGN);
        plan = tpb::plan_splits(tiles, P.k_stages, pieces, tiled, sms, a->workspace_bytes, M);
    }
    P.splits = plan.splits;
    P.stages_per_split = plan.stages_per_split;
    P.counters = static_cast<unsigned int*>(a->workspace);
    P.out = qkv ? a->qkv_q_out : a->out;
    P.ldo = qkv ? a->qkv_ldq : a->ldo;
    P.k_rows = static_cast<__nv_bfloat16*>(a->qkv_k_rows);
    P.v_rows = static_cast<__nv_bfloat16*>(a->qkv_v_rows);
    P.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(a->workspace) + tpb::kCounterBytes);
    const int grid = std::min(tiles * plan.splits, sms);
    TPB_REQUIRE((a->flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    // the second epilogue group (warps 6..9) only has work in unsplit launches with the plain epilogue
    const bool two_groups = P.epilogue == tpb::kEpiPlain && P.splits == 1;
    cfg.blockDim = dim3(two_groups ? tpb::kThreads : tpb::kThreads - 128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (a->flags & TPB200_FLAG_PDL) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    // A split launch's CTAs wait for the partner CTAs of their tile, so all of them must be resident together.
    // The grid never exceeds one CTA per SM, but another kernel holding SMs at the same time (a launch on another
    // stream) could keep partners out: a cooperative launch is placed only when the whole grid fits.
    if (plan.splits > 1) {
        attr[nattr].id = cudaLaunchAttributeCooperative;
        attr[nattr].val.cooperative = 1;
        ++nattr;
    }
    if (nattr > 0) {
        cfg.attrs = attr;
        cfg.numAttrs = nattr;
    }
#ifdef TPB_TIMELINE
    static std::atomic<int> launch_no{0};
    P.debug_slot = launch_no.fetch_add(1);
#endif
    const cudaError_t err = tiled ? cudaLaunchKernelEx(&cfg, tpb::nvfp4_gemm_kernel<true>, P)
                                  : cudaLaunchKernelEx(&cfg, tpb::nvfp4_gemm_kernel<false>, P);
    if (err != cudaSuccess) return TPB200_ERR_CUDA;
    return tpb_launch_status();
}

extern "C" int tpb200_nvfp4_gemm(const void* a_packed, int a_pitch, const void* a_sf, const void* b_packed,
                                 int b_pitch, const void* b_sf, float alpha, const void* bias_f32, int activation,
                                 void* out, int out_dtype, int ldo, int M, int N, int K, int flags,
                                 tpb200_stream_t stream) {
    TPB_REQUIRE(flags == TPB200_FLAG_NONE, TPB200_ERR_ENUM);
    tpb200_nvfp4_gemm_args a = {};
    a.a_packed = a_packed; a.a_pitch = a_pitch; a.a_sf = a_sf; a.a_pieces = 1;
    a.b_packed = b_packed; a.b_pitch = b_pitch; a.b_sf = b_sf;
    a.alpha = alpha; a.bias = static_cast<const float*>(bias_f32); a.activation = activation;
    a.out = out; a.out_dtype = out_dtype; a.ldo = ldo;
    a.M = M; a.N = N; a.K = K;
    return tpb200_nvfp4_gemm_ex(&a, stream);
}

#ifdef TPB_TIMELINE
// Diagnostic build only: the stamps of the last launches ([slot][CTA][point], nanoseconds).
extern "C" int tpb200_debug_gemm_timeline(unsigned long long* out, size_t bytes) {
    if (bytes > sizeof(tpb::g_gemm_timeline)) bytes = sizeof(tpb::g_gemm_timeline);
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, tpb::g_gemm_timeline, bytes);
    return 0;
}
#endif

extern "C" int tpb200_measure_fp4_mma_rate(int mmas_per_cta, tpb200_stream_t stream) {
    TPB_REQUIRE(mmas_per_cta >= 1 && mmas_per_cta <= (1 << 22), TPB200_ERR_SHAPE);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    const int smem = 3 * tpb::kTile + 3 * tpb::kSfSlab + 64 + 1024;
    if (cudaFuncSetAttribute(tpb::fp4_mma_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    tpb::fp4_mma_rate_kernel<<<sms, 64, smem, reinterpret_cast<cudaStream_t>(stream)>>>(mmas_per_cta);
    return tpb_launch_status();
}
