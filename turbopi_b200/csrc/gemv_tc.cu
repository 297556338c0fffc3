// Decode-shaped (M <= 16 tokens) NVFP4 weight-only GEMV on the tensor cores.
//
// The CUDA-core GEMV is bound by instruction issue (decode + FMA per weight); here the SM does
// no per-weight work at all.  The roles of a GEMM are swapped: a 128-row slab of the WEIGHT
// matrix is the A operand of tcgen05.mma kind::mxf4nvf4, the activations are the B operand.
// bf16 activations keep their precision as residual e2m1 pieces (see nvfp4_gemm.cu) stacked
// along N: piece p of token t is B row 16 p + t, so one MMA (N = 16 * pieces) per 64-wide K
// atom handles all pieces and the epilogue adds the pieces' columns.
//
// Weights are stored PRE-TILED in the shared-memory image of the 128-byte swizzle, scales included:
// the tensor-core GEMM's B image (tpb200_nvfp4_tile_weights), block (n_blk, ks) of 36 KB = 256 rows x
// 128 B of codes (16-byte chunk c of row r at c ^ (r & 7)) + the two 2 KB scale slabs; one image
// serves the prefill GEMM and this decode GEMV.  A stage = one such block (four plain 1-D bulk copies
// issued side by side) + the activation block of the same K range (16 * pieces rows x 128 B of codes
// in the same pattern + one 2 KB scale slab), feeding two MMAs per 64-wide K atom (weight rows 0..127
// and 128..255, two accumulators).  A ring of five stages keeps the stream going.
//
// The activation block comes from one of two places:
//   fused      four warps of the CTA quantise the K range of the raw [M, K] activations straight into
//              the stage buffer while the weight block is in flight (row amax -> power-of-two pre-scale
//              -> residual pieces; the same arithmetic as the stand-alone quantiser), so a decode step
//              is ONE launch;
//   pre-tiled  a fifth bulk copy from an image written by tpb200_nvfp4_quantize_act(s)_tc.
//
// Schedule.  The host plans every launch: a work unit is (problem, 256-row tile, K range); whole
// tiles are dealt to the CTAs longest-first so that no partial sums cross CTAs, and only when a launch
// has too few or too long tiles for the machine are tiles cut along K.  A cut tile's pieces write their
// partial sums (valid tokens only) to caller-provided scratch and the CTA that arrives last on the tile's
// counter adds them in K order (deterministic), applies the epilogue and resets the counter.  Nothing
// ever waits on another CTA.  The unit list travels in the kernel's parameter space.
#include <algorithm>
#include <atomic>

#include "tcgen05.cuh"

namespace tpb {
namespace {

constexpr int kMaxStages = 6;
constexpr int kWTile = 128 * 128;     // codes of 128 weight rows for one K stage
constexpr int kSfSlab = 2048;         // 4 scale atoms
constexpr int kWBlock = 2 * (kWTile + kSfSlab);   // 256 rows: [codes 32 KB][slab rows 0..127][slab rows 128..255]
constexpr int kMaxNB = 64;            // 16 tokens x 4 pieces
// a stage holds one weight block and one activation block (16 * pieces rows + scale slab); the ring
// takes as many stages as fit: 5 for up to 3 pieces, 4 for 4
__host__ __device__ constexpr int stage_bytes(int pieces) { return kWBlock + 16 * pieces * 128 + kSfSlab; }
__host__ __device__ constexpr int num_stages(int pieces) {
    return (227 * 1024 - 3072) / stage_bytes(pieces) < kMaxStages ? (227 * 1024 - 3072) / stage_bytes(pieces) : kMaxStages;
}
// warps: 0 producer, 1 MMA issuer, 2..5 epilogue, 6 scale copier, 7..10 activation quantisers
constexpr int kThreads = 352;
constexpr int kActWarp0 = 7;
constexpr int kTmemCols = 512;
// tensor memory: accumulator (buffer b, row half h) at column b * 128 + h * 64, then the scales
// two sets of scale columns (stages alternate): 32 for the weights' two row halves + 16 for the activations
constexpr uint32_t kSfSetCols = 48;
constexpr uint32_t kSfaCol = 256;
constexpr uint32_t kSfbCol = kSfaCol + 32;
constexpr int kMaxProblems = TPB200_MAX_GROUP;
constexpr int kMaxCtas = 256;
constexpr int kRsRing = 16;           // row multipliers of the units in flight between quantiser and epilogue
constexpr int kSlotFloats = 16 * 256; // partial sums of one unit: [token][row of the tile]

struct TcProblem {
    const uint8_t* w_image;     // [row_tiles of 256][k_stages][36864]
    const void* x;              // fused: raw activations [M, ldx]; pre-tiled: [k_stages][NB * 128 + 2048]
    const float* row_scale;     // pre-tiled only: [M]
    const void* bias;
    void* out;
    int N, K;
    int ldo, ldx;
    float global_scale;
    int k_stages;
};

// One work unit of a CTA: K stages [ks0, ks1) of row tile rt of problem p, accumulated in tensor memory
// as one K range.
struct TcUnit {
    uint8_t p;
    uint8_t shared;      // the tile is cut along K: hand the partial sums over
    uint16_t rt;
    uint16_t ks0, ks1;
    uint16_t slot0;      // first partial-sum slot of the tile
    uint16_t counter;    // the tile's arrival counter
    uint8_t slot;        // this unit's slot, in K order
    uint8_t nslots;      // units the tile was cut into
    uint16_t pad;
};
static_assert(sizeof(TcUnit) == 16, "unit records are copied as 16-byte words");

template <int kMaxUnits>
struct TcParams {
    int num_problems;
    int M;
    int pieces;
    int x_dtype, bias_dtype, out_dtype, activation;
    int fused;
    int debug_slot;             // diagnostic builds: which timeline slot this launch writes
    int pool_begin, pool_size;  // units[pool_begin, pool_begin + pool_size) are drawn by whichever CTA is free
    unsigned int* queue;        // the pool's ticket counter (zero between launches)
    float* scratch;
    int* counters;
    TcProblem prob[kMaxProblems];
    uint16_t cta_begin[kMaxCtas + 1];
    TcUnit units[kMaxUnits];
};

constexpr int kUnitRing = 16;         // work units in flight between the producer and the slowest role of a CTA
constexpr uint8_t kEndOfUnits = 0xFF; // `p` of the record that closes a CTA's unit list

struct SharedControl {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sf_full[2];      // scale set j copied into tensor memory (arrives through tcgen05.commit)
    uint64_t sf_empty[2];     // the MMAs that read scale set j are done
    uint32_t tmem_base;
    volatile int abort_flag;
    int ticket;
    volatile int units_published;
    TcUnit units[kUnitRing];              // the CTA's unit list as the producer publishes it
    float row_scale[kRsRing][16];
    int act_e[4][2][16];                  // per quantiser warp: pre-scale exponents of its two cached tensors
};

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Power-of-two pre-scale that brings a row's largest magnitude into [1024, 2048): the block scales of the
// pieces then sit in the upper range of UE4M3.  Returns the exponent e (pre-scale 2^e, undone by 2^-e).
// 16 consecutive elements, already in registers as loaded (two 16-byte words of 16-bit elements, or four of fp32)
__device__ __forceinline__ void unpack16(const uint4 (&raw)[4], int dtype, float (&v)[16]) {
    if (dtype == TPB200_F32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[4 * i] = __uint_as_float(raw[i].x);
            v[4 * i + 1] = __uint_as_float(raw[i].y);
            v[4 * i + 2] = __uint_as_float(raw[i].z);
            v[4 * i + 3] = __uint_as_float(raw[i].w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = dtype == TPB200_F16 ? __half22float2(*reinterpret_cast<const __half2*>(&w[j]))
                                                     : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                v[8 * i + 2 * j] = f.x;
                v[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
}

// Unit i of this CTA's list, once the producer has published it.  False at the end of the list, after an
// abort, or when the (bounded) wait runs out.
__device__ __forceinline__ bool fetch_unit(SharedControl* ctl, int i, TcUnit& un) {
    if (ctl->units_published <= i) {
        const long long start = clock64();
        while (ctl->units_published <= i) {
            if (ctl->abort_flag) return false;
            if (clock64() - start > 2000000000LL) {
                record_error(kErrGemvUnitQueueTimeout);
                ctl->abort_flag = 1;
                return false;
            }
        }
    }
    uint32_t w0, w1, w2, w3;
    asm volatile("ld.volatile.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                 : "r"(smem_u32(&ctl->units[i & (kUnitRing - 1)]))
                 : "memory");
    uint4 w = make_uint4(w0, w1, w2, w3);
    un = *reinterpret_cast<TcUnit*>(&w);
    return un.p != kEndOfUnits;
}

// the same for a whole warp: lane 0 waits, every lane gets the record
__device__ __forceinline__ bool fetch_unit_warp(SharedControl* ctl, int i, int lane, TcUnit& un) {
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    int ok = 0;
    if (lane == 0) {
        TcUnit t;
        ok = fetch_unit(ctl, i, t) ? 1 : 0;
        w = *reinterpret_cast<uint4*>(&t);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    w.x = __shfl_sync(0xffffffffu, w.x, 0);
    w.y = __shfl_sync(0xffffffffu, w.y, 0);
    w.z = __shfl_sync(0xffffffffu, w.z, 0);
    w.w = __shfl_sync(0xffffffffu, w.w, 0);
    un = *reinterpret_cast<TcUnit*>(&w);
    return ok != 0;
}

#ifdef TPB_TIMELINE
// Diagnostic build only (-DTPB_TIMELINE): every CTA of the last launches leaves globaltimer stamps of its
// milestones here; tpb200_debug_gemv_tc_timeline() copies them out.
constexpr int kTlSlots = 4, kTlPoints = 16;
__device__ unsigned long long g_timeline[kTlSlots][kMaxCtas][kTlPoints];
__device__ __forceinline__ unsigned long long tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define TL(point) g_timeline[P.debug_slot & (kTlSlots - 1)][blockIdx.x][point] = tl_now()
#else
#define TL(point) ((void)0)
#endif

template <int kMaxUnits>
__global__ void __launch_bounds__(kThreads, 1) nvfp4_gemv_tc_kernel(const __grid_constant__ TcParams<kMaxUnits> P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int kStages = num_stages(P.pieces);
    const int kStageBytes = stage_bytes(P.pieces);
    SharedControl* ctl = reinterpret_cast<SharedControl*>(smem + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int NB = 16 * P.pieces;
    const int u_lo = P.cta_begin[blockIdx.x];        // this CTA's fixed units; more may come from the shared pool
    const int u_hi = P.cta_begin[blockIdx.x + 1];
    const bool fused = P.fused != 0;

    if (threadIdx.x == 0) {
        TL(0);
        for (int s = 0; s < kMaxStages; ++s) {
            // a stage is full when its weight block has landed (one arrival with the byte count) and,
            // in the fused form, when the quantiser warp that owns the stage has written the activations
            mbar_init(&ctl->full[s], fused ? 2 : 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);
            mbar_init(&ctl->sf_full[b], 1);
            mbar_init(&ctl->sf_empty[b], 1);
        }
        ctl->abort_flag = 0;
        ctl->units_published = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tc::tmem_alloc(&ctl->tmem_base, kTmemCols);
        tc::tmem_relinquish();
    }
    if (fused && warp >= kActWarp0) {
        // rows of tokens >= M are never written again: they stay zero codes with zero scales
        const int at = threadIdx.x - kActWarp0 * 32;
        const int abytes = NB * 128 + kSfSlab;
        for (int s = 0; s < kStages; ++s) {
            uint4* a = reinterpret_cast<uint4*>(smem + s * kStageBytes + kWBlock);
            for (int i = at; i < abytes / 16; i += 128) a[i] = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
    }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = ctl->tmem_base;
    pdl_launch_dependents();
    if (threadIdx.x == 0) TL(1);

    if (warp == 0) {
        // ------------------------------------------------------------ producer (whole warp): lane 0 owns the
        // barrier hand-shakes and the unit list, lanes 0..3 each copy a quarter of the stage's weight block and
        // lane 4 the pre-tiled activation block.  (A thread that issues a bulk copy is held for ~0.3 us whatever
        // the size; requests issued side by side from several lanes overlap that.)  Weights never depend on the
        // previous kernel, so the first stages' weight blocks are requested before griddepcontrol.wait;
        // activations are written by the previous kernel.
        //
        // Unit list: the CTA's fixed units first, then units drawn from the launch's shared pool (one atomic
        // per unit on a counter that the last drawer returns to zero).  SMs do not get equal shares of the
        // memory system; with fixed lists alone the slowest CTA finishes microseconds after the others and
        // holds up the next kernel of the stream.  The pool is touched only after griddepcontrol.wait, when
        // the previous launch on this workspace has left its counter at zero.
        const uint32_t xbytes = fused ? 0u : static_cast<uint32_t>(NB) * 128u + kSfSlab;
        constexpr uint32_t kQuarter = kWBlock / 4;
        int published = 0;
        auto publish = [&](const TcUnit& un) {
            if (lane == 0) {
                ctl->units[published & (kUnitRing - 1)] = un;
                __threadfence_block();
                ctl->units_published = published + 1;
            }
            ++published;
        };
        TcUnit end_mark = {};
        end_mark.p = kEndOfUnits;

        // The first unit is announced before anything else: the other roles (the quantiser warps above all) start
        // on it while this warp is still held by the copy requests below.
        int next_fixed = u_lo;
        TcUnit cur = end_mark;
        bool have_cur = false;
        if (next_fixed < u_hi) {
            cur = P.units[next_fixed++];
            have_cur = true;
            publish(cur);
        }
        // the ring's first fill goes out in ONE round: lane l requests quarter l % 4 of stage l / 4
        int pre = 0;
        const uint8_t* my_src = nullptr;
        for (int u = u_lo; u < u_hi && pre < kStages; ++u) {
            const TcUnit un = P.units[u];
            const TcProblem& pr = P.prob[un.p];
            for (int ks = un.ks0; ks < un.ks1 && pre < kStages; ++ks, ++pre) {
                const size_t blk = static_cast<size_t>(un.rt) * pr.k_stages + ks;
                if ((lane >> 2) == pre) my_src = pr.w_image + blk * kWBlock + (lane & 3) * kQuarter;
            }
        }
        if (lane < pre) mbar_expect_tx(&ctl->full[lane], kWBlock + xbytes);
        __syncwarp();
        const uint64_t stream_once = l2_policy_evict_first();   // weights pass through L2 once
        if (my_src != nullptr) {
            bulk_copy_g2s_hint(smem + (lane >> 2) * kStageBytes + (lane & 3) * kQuarter, my_src, kQuarter,
                               &ctl->full[lane >> 2], stream_once);
        }
        if (lane == 0) TL(2);
        pdl_wait_prior_grids();
        if (lane == 0) TL(3);
        bool pool_open = P.pool_size > 0;
        // one draw from the pool; the drawer of the last ticket (every CTA fails exactly once) re-arms the counter
        auto draw = [&](TcUnit& un) -> bool {
            unsigned int ticket = 0;
            if (lane == 0) ticket = atomicAdd(P.queue, 1u);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket < static_cast<unsigned int>(P.pool_size)) {
                un = P.units[P.pool_begin + ticket];
                return true;
            }
            pool_open = false;
            if (lane == 0 && ticket == static_cast<unsigned int>(P.pool_size) + gridDim.x - 1u) {
                atomicExch(P.queue, 0u);
            }
            return false;
        };
        if (!have_cur && pool_open) {
            have_cur = draw(cur);
            if (have_cur) publish(cur);
        }
        int it = 0;
        bool stop = false;
        while (have_cur && !stop) {
            const TcUnit un = cur;
            const TcProblem& pr = P.prob[un.p];
            for (int ks = un.ks0; ks < un.ks1; ++ks, ++it) {
                const int s = it % kStages;
                uint8_t* st = smem + s * kStageBytes;
                const size_t blk = static_cast<size_t>(un.rt) * pr.k_stages + ks;
                int bad = 0;
                if (lane == 0) {
                    if (ctl->abort_flag) {
                        bad = 1;
                    } else if (it >= pre) {
                        if (it >= kStages && !mbar_wait_bounded(&ctl->empty[s], ((it / kStages) - 1) & 1)) {
                            record_error(kErrGemmEmptyBarrierTimeout);
                            ctl->abort_flag = 1;
                            bad = 1;
                        } else {
                            mbar_expect_tx(&ctl->full[s], kWBlock + xbytes);
                        }
                    }
                }
                bad = __shfl_sync(0xffffffffu, bad, 0);
                if (bad) {
                    stop = true;
                    break;
                }
                if (lane < 4) {
                    if (it >= pre) {
                        bulk_copy_g2s_hint(st + lane * kQuarter, pr.w_image + blk * kWBlock + lane * kQuarter, kQuarter,
                                           &ctl->full[s], stream_once);
                    }
                } else if (lane == 4 && !fused) {
                    bulk_copy_g2s(st + kWBlock, static_cast<const uint8_t*>(pr.x) + static_cast<size_t>(ks) * xbytes, xbytes,
                                  &ctl->full[s]);
                }
            }
            if (stop) break;
            // The next unit is drawn only now, not ahead of time: the ticket's round trip passes while the ring
            // (five stages deep) still feeds the MMAs, and a slow CTA holds one unit less when the pool runs dry.
            have_cur = false;
            if (next_fixed < u_hi) {
                cur = P.units[next_fixed++];
                have_cur = true;
            } else if (pool_open) {
                have_cur = draw(cur);
            }
            if (have_cur) publish(cur);
        }
        publish(end_mark);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = tc::make_idesc_mxf4nvf4(NB);
            // descriptor words: (stage address >> 4) + constants; see tcgen05.cuh
            const uint32_t base16 = smem_u32(smem) >> 4;
            const uint32_t stage16 = static_cast<uint32_t>(kStageBytes) >> 4;
            const uint32_t t_sfa = tmem_base + kSfaCol;
            const uint32_t t_sfb = tmem_base + kSfbCol;
            int s = 0;
            uint32_t full_phase = 0;
            uint32_t lo0 = base16;
            uint32_t g = 0;                        // stages issued so far; stage g uses scale set g & 1
            TcUnit un;
            for (int i = 0; !ctl->abort_flag && fetch_unit(ctl, i, un); ++i) {
                const int buf = i & 1;
                if (i >= 2 && !mbar_wait_bounded(&ctl->acc_empty[buf], ((i >> 1) - 1) & 1)) {
                    record_error(kErrGemmEpilogueBarrierTimeout);
                    ctl->abort_flag = 1;
                    break;
                }
                tc::fence_after_thread_sync();
                const uint32_t tmem_acc = tmem_base + buf * 128;
                uint32_t accumulate = 0;
                for (int ks = un.ks0; ks < un.ks1; ++ks) {
                    if (!mbar_wait_bounded(&ctl->full[s], full_phase)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        ctl->abort_flag = 1;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    if (g == 0) TL(4);
                    // the scale copier (warp 6) has moved this stage's scales into set g & 1
                    const uint32_t set = g & 1u;
                    if (!mbar_wait_bounded(&ctl->sf_full[set], (g >> 1) & 1u)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        ctl->abort_flag = 1;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    const uint32_t sfa = t_sfa + set * kSfSetCols;
                    const uint32_t sfb = t_sfb + set * kSfSetCols;
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        const uint64_t xdesc = tc::desc_from_words(lo0 + ((kWBlock + a * 32) >> 4), tc::kDescHiKmajorSw128);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            tc::mma_mxf4nvf4(tmem_acc + h * kMaxNB,
                                             tc::desc_from_words(lo0 + ((h * kWTile + a * 32) >> 4), tc::kDescHiKmajorSw128),
                                             xdesc, idesc, sfa + 16 * h + 4 * a, sfb + 4 * a, a == 0 ? accumulate : 1u);
                        }
                    }
                    accumulate = 1;
                    tc::commit(&ctl->empty[s]);
                    tc::commit(&ctl->sf_empty[set]);
                    ++g;
                    if (++s == kStages) {
                        s = 0;
                        full_phase ^= 1;
                        lo0 = base16;
                    } else {
                        lo0 += stage16;
                    }
                }
                tc::commit(&ctl->acc_full[buf]);
            }
            TL(5);
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ scale copier.
        // One thread issues every tcgen05 instruction it is given at ~60 cycles apiece; with the 12 scale
        // copies of a stage on the MMA thread that thread, not the weight stream, set the pace.  Here they
        // run one stage ahead into the other set of scale columns.  The copies do not depend on the tile, so
        // this lane only needs the number of stages of each unit.
        if (lane == 0) {
            const uint32_t base16 = smem_u32(smem) >> 4;
            const uint32_t stage16 = static_cast<uint32_t>(kStageBytes) >> 4;
            const uint32_t off_sfb16 = static_cast<uint32_t>(kWBlock + NB * 128) >> 4;
            int s = 0;
            uint32_t full_phase = 0, lo0 = base16;
            int g = 0;
            TcUnit un;
            bool stop = false;
            for (int i = 0; !stop && !ctl->abort_flag && fetch_unit(ctl, i, un); ++i) {
                for (int ks = un.ks0; ks < un.ks1; ++ks, ++g) {
                    const uint32_t set = g & 1;
                    if (!mbar_wait_bounded(&ctl->full[s], full_phase) ||
                        (g >= 2 && !mbar_wait_bounded(&ctl->sf_empty[set], ((g >> 1) - 1) & 1))) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        ctl->abort_flag = 1;
                        stop = true;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    const uint32_t sfa = tmem_base + kSfaCol + set * kSfSetCols;
                    const uint32_t sfb = tmem_base + kSfbCol + set * kSfSetCols;
                    // stage: [codes rows 0..127][codes rows 128..255][slab 0..127][slab 128..255][x codes][x slab]
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        tc::cp_sf_32x128b(sfa + 4 * a, tc::desc_from_words(lo0 + ((2 * kWTile + a * 512) >> 4), tc::kDescHiSfAtom));
                        tc::cp_sf_32x128b(sfa + 16 + 4 * a,
                                          tc::desc_from_words(lo0 + ((2 * kWTile + kSfSlab + a * 512) >> 4), tc::kDescHiSfAtom));
                        tc::cp_sf_32x128b(sfb + 4 * a, tc::desc_from_words(lo0 + off_sfb16 + ((a * 512) >> 4), tc::kDescHiSfAtom));
                    }
                    tc::commit(&ctl->sf_full[set]);
                    if (++s == kStages) {
                        s = 0;
                        full_phase ^= 1;
                        lo0 = base16;
                    } else {
                        lo0 += stage16;
                    }
                }
            }
        }
    } else if (warp >= kActWarp0) {
        // ------------------------------------------------------------ activation quantisers (fused form).
        // Quantiser warp w owns every fourth stage of the CTA's stage sequence (stage number % 4 == w): for
        // such a stage it turns the 256-wide K slice of all M token rows into residual pieces inside the stage
        // buffer and arrives on the stage's `full` barrier.  Four stages are in work at once, so the latency
        // of the activation loads and the ~0.6 us of arithmetic per stage stay off the weight stream's
        // pace (0.55 us per stage).  Row pre-scales come from one pass over the tensor, kept per warp for its
        // two most recent activation tensors.  The warps never talk to each other, so each can leave on its
        // own if a wait runs out.
        if (fused) {
            const int aw = warp - kActWarp0;
            const void* cache_x0 = nullptr;
            const void* cache_x1 = nullptr;
            int victim = 0;
            // The activations come from the previous kernel, so they may only be READ after griddepcontrol.wait.
            // Asking the L2 for their lines before that is harmless (the L2 is the point of coherence: a line
            // written later is simply updated) and takes the DRAM round trip -- two microseconds while the weight
            // streams of two launches saturate the memory system -- out of the path to the first MMA.
            if (u_lo < u_hi) {
                const TcUnit first_unit = P.units[u_lo];
                const TcProblem& fp = P.prob[first_unit.p];
                const int row_bytes = fp.K * (P.x_dtype == TPB200_F32 ? 4 : 2);
                const int lines = (row_bytes + 127) >> 7;
                for (int t = 0; t < P.M; ++t) {
                    const char* row = static_cast<const char*>(fp.x) + static_cast<size_t>(t) * fp.ldx * (P.x_dtype == TPB200_F32 ? 4 : 2);
                    for (int ln = aw * 32 + lane; ln < lines; ln += 128) {
                        asm volatile("prefetch.global.L2 [%0];" ::"l"(row + (static_cast<size_t>(ln) << 7)));
                    }
                }
            }
            pdl_wait_prior_grids();
            if (aw == 0 && lane == 0) TL(8);
            int it = 0;                                                 // stages of the units seen so far
            bool stop = false;
            TcUnit un;
            for (int i = 0; !stop && fetch_unit_warp(ctl, i, lane, un); ++i) {
                if (aw == 0 && lane == 0 && i == 0) TL(12);
                const int nst = un.ks1 - un.ks0;
                const int first = (aw - it) & 3;                        // this warp's first stage inside the unit
                if (first < nst) {
                    const TcProblem& pr = P.prob[un.p];
                    const void* x = pr.x;
                    const int ldx = pr.ldx;
                    const int nblk = pr.K >> 4;
                    int slot;
                    bool need_amax = false;
                    if (cache_x0 == x) {
                        slot = 0;
                    } else if (cache_x1 == x) {
                        slot = 1;
                    } else {
                        slot = victim;
                        victim ^= 1;
                        if (slot == 0) cache_x0 = x;
                        else cache_x1 = x;
                        need_amax = true;          // done below, behind the first stage's loads
                    }
                    const int* e_row = ctl->act_e[aw][slot];
                    bool scale_pending = first == 0;   // the owner of the unit's first stage publishes the row multipliers
                    for (int o = first; o < nst && !stop; o += 4) {
                        const int ks = un.ks0 + o;
                        const int git = it + o;
                        const int s = git % kStages;
                        uint8_t* blk = smem + s * kStageBytes + kWBlock;
                        bool waited = false;
                        // one round per token row: lane = (16-element block of the stage, half of that block); the two
                        // lanes of a block share its maximum through one shuffle, so a block's three residual pieces are
                        // a chain of 8-element steps instead of 16-element ones
                        const int kbl = lane >> 1, hb = lane & 1;          // block inside the stage, half of the block
                        for (int t = 0; t < P.M; ++t) {
                            uint4 raw[2];
                            const int kb = ks * 16 + kbl;
                            const bool valid = kb < nblk;
                            if (valid) {
                                const size_t e0 = static_cast<size_t>(t) * ldx + static_cast<size_t>(kb) * 16 + hb * 8;
                                if (P.x_dtype == TPB200_F32) {
                                    const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const float*>(x) + e0);
                                    raw[0] = __ldg(gp);
                                    raw[1] = __ldg(gp + 1);
                                } else {
                                    raw[0] = __ldg(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + e0));
                                }
                            }
                            if (need_amax) {
                                // a new activation tensor: its row maxima, with the stage's loads already in flight
                                need_amax = false;
                                for (int t = 0; t < P.M; ++t) {
                                    // every block of a lane's share is requested before the first is used (eight
                                    // blocks per lane and round for 16-bit activations, four for fp32): a row of up
                                    // to 4096 elements costs ONE memory latency, at a time when the memory system
                                    // is saturated by the weight stream and a round trip takes well over a microsecond
                                    float amax = 0.0f;
                                    const bool wide = P.x_dtype == TPB200_F32;
                                    const int per_round = wide ? 4 : 8;
                                    for (int kb0 = 0; kb0 < nblk; kb0 += 32 * per_round) {
                                        uint4 araw[16];
#pragma unroll
                                        for (int j = 0; j < 8; ++j) {
                                            const int kb = kb0 + lane + 32 * j;
                                            if (j < per_round && kb < nblk) {
                                                const size_t e0 = static_cast<size_t>(t) * ldx + static_cast<size_t>(kb) * 16;
                                                if (wide) {
                                                    const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const float*>(x) + e0);
#pragma unroll
                                                    for (int w = 0; w < 4; ++w) araw[(4 * j + w) & 15] = __ldg(gp + w);
                                                } else {
                                                    const uint4* gp = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + e0);
                                                    araw[2 * j] = __ldg(gp);
                                                    araw[2 * j + 1] = __ldg(gp + 1);
                                                }
                                            }
                                        }
#pragma unroll
                                        for (int j = 0; j < 8; ++j) {
                                            if (j < per_round && kb0 + lane + 32 * j < nblk) {
                                                uint4 blk4[4];
                                                if (wide) {
#pragma unroll
                                                    for (int w = 0; w < 4; ++w) blk4[w] = araw[(4 * j + w) & 15];
                                                } else {
                                                    blk4[0] = araw[2 * j];
                                                    blk4[1] = araw[2 * j + 1];
                                                    blk4[2] = blk4[3] = make_uint4(0u, 0u, 0u, 0u);
                                                }
                                                float r[16];
                                                unpack16(blk4, P.x_dtype, r);
#pragma unroll
                                                for (int q = 0; q < 16; ++q) amax = fmaxf(amax, fabsf(r[q]));
                                            }
                                        }
                                    }
#pragma unroll
                                    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                                    if (lane == 0) ctl->act_e[aw][slot][t] = prescale_exponent(amax);
                                }
                                __syncwarp();
                            }
                            if (aw == 0 && lane == 0 && git == 0) TL(13);
                            if (scale_pending) {
                                // the epilogue of this unit multiplies by 2^-e
                                scale_pending = false;
                                if (lane < P.M) ctl->row_scale[i & (kRsRing - 1)][lane] = ldexpf(1.0f, -e_row[lane]);
                            }
                            if (!waited) {
                                waited = true;
                                int bad = 0;
                                if (lane == 0) {
                                    if (ctl->abort_flag) {
                                        bad = 1;
                                    } else if (git >= kStages && !mbar_wait_bounded(&ctl->empty[s], ((git / kStages) - 1) & 1)) {
                                        record_error(kErrGemmEmptyBarrierTimeout);
                                        ctl->abort_flag = 1;
                                        bad = 1;
                                    }
                                }
                                bad = __shfl_sync(0xffffffffu, bad, 0);
                                if (bad) {
                                    stop = true;
                                    break;
                                }
                            }
                            float r[8];
#pragma unroll
                            for (int w = 0; w < 8; ++w) r[w] = 0.0f;
                            if (valid) {
                                if (P.x_dtype == TPB200_F32) {
                                    r[0] = __uint_as_float(raw[0].x); r[1] = __uint_as_float(raw[0].y);
                                    r[2] = __uint_as_float(raw[0].z); r[3] = __uint_as_float(raw[0].w);
                                    r[4] = __uint_as_float(raw[1].x); r[5] = __uint_as_float(raw[1].y);
                                    r[6] = __uint_as_float(raw[1].z); r[7] = __uint_as_float(raw[1].w);
                                } else {
                                    const uint32_t w4[4] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w};
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        const float2 f = P.x_dtype == TPB200_F16
                                                             ? __half22float2(*reinterpret_cast<const __half2*>(&w4[j]))
                                                             : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w4[j]));
                                        r[2 * j] = f.x;
                                        r[2 * j + 1] = f.y;
                                    }
                                }
                                const float pre = ldexpf(1.0f, e_row[t]);
#pragma unroll
                                for (int w = 0; w < 8; ++w) r[w] *= pre;
                            }
                            const int c = kbl >> 1;                    // 16-byte chunk of the 128-byte row
                            for (int pc = 0; pc < P.pieces; ++pc) {
                                const int prow = pc * 16 + t;
                                uint8_t* dst = blk + prow * 128 + ((c ^ (prow & 7)) << 4) + (kbl & 1) * 8 + hb * 4;
                                uint8_t* sf_dst = blk + NB * 128 + (kbl >> 2) * 512 + (prow & 31) * 16 + ((prow >> 5) & 3) * 4 + (kbl & 3);
                                uint32_t word;
                                const uint8_t code = quantize_half8_piece(r, word);   // zeros in, zero code and scale out
                                if (hb == 0) *sf_dst = code;
                                *reinterpret_cast<uint32_t*>(dst) = word;
                            }
                        }
                        if (stop) break;
                        if (aw == 0 && lane == 0 && git == 0) TL(14);
                        fence_proxy_async_smem();                      // the tensor core reads these bytes
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->full[s]);
                        if (aw == 0 && lane == 0 && git == 0) TL(9);
                    }
                }
                it += nst;
            }
            if (aw == 0 && lane == 0) TL(10);
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
        const int q = warp & 3;
        const int et = q * 32 + lane;            // 0..127: the weight row inside the tile
        pdl_wait_prior_grids();                   // the output buffer may still be read by the previous kernel
        TcUnit un;
        for (int i = 0; !ctl->abort_flag && fetch_unit_warp(ctl, i, lane, un); ++i) {
            const TcProblem& pr = P.prob[un.p];
            const int buf = i & 1;
            if (!mbar_wait_bounded(&ctl->acc_full[buf], (i >> 1) & 1)) {
                record_error(kErrGemmMmaBarrierTimeout);
                ctl->abort_flag = 1;
                break;
            }
            tc::fence_after_thread_sync();
            if (warp == 2 && lane == 0) TL(11);
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 128;
            float v[2][16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                // all pieces of a row half are requested before the one wait (a tensor-memory load takes a few
                // hundred nanoseconds; one after the other they cost more than the unit's MMAs)
                uint32_t r[4][16];
#pragma unroll
                for (int pc = 0; pc < 4; ++pc) {
                    if (pc < P.pieces) tmem_ld_32x32b_x16(taddr + h * kMaxNB + pc * 16, r[pc]);
                }
                tc::tmem_ld_wait();
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                    if (t >= P.M) break;
                    float acc = __uint_as_float(r[0][t]);
#pragma unroll
                    for (int pc = 1; pc < 4; ++pc) {
                        if (pc < P.pieces) acc += __uint_as_float(r[pc][t]);
                    }
                    v[h][t] = acc;
                }
            }
            tc::fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);

            bool finalize = true;
            if (un.shared) {
                // this unit covers only part of the tile's K range: hand its sums over
                float* part = P.scratch + static_cast<size_t>(un.slot0) * kSlotFloats;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        if (t < P.M) part[(static_cast<size_t>(un.slot) * 16 + t) * 256 + h * 128 + et] = v[h][t];
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) ctl->ticket = atomicAdd(P.counters + un.counter, 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finalize = (ctl->ticket == un.nslots - 1);
                if (finalize) {
                    __threadfence();
                    if (P.M == 1) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            float acc = 0.0f;
                            for (int sl = 0; sl < un.nslots; ++sl) {
                                acc += __ldcg(part + static_cast<size_t>(sl) * kSlotFloats + h * 128 + et);
                            }
                            v[h][0] = acc;
                        }
                    } else {
                        // several tokens: slot by slot (the sum keeps its K order) with all of a slot's loads in
                        // flight together -- token by token the walk is a chain of M * slots L2 round trips
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
#pragma unroll
                            for (int t = 0; t < 16; ++t) v[h][t] = 0.0f;
                        }
#pragma unroll 2
                        for (int sl = 0; sl < un.nslots; ++sl) {
                            const float* src = part + static_cast<size_t>(sl) * kSlotFloats + et;
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
#pragma unroll
                                for (int t = 0; t < 16; ++t) {
                                    if (t < P.M) v[h][t] += __ldcg(src + t * 256 + h * 128);
                                }
                            }
                        }
                    }
                    if (et == 0) P.counters[un.counter] = 0;               // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");              // ticket slot free for the next unit
            }
            if (finalize) {
                // the row multipliers were written by a quantiser warp before it released the unit's first
                // stage, which the MMAs behind this accumulator have consumed
                const float* rs = fused ? ctl->row_scale[i & (kRsRing - 1)] : pr.row_scale;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int n = un.rt * 256 + h * 128 + et;
                    if (n >= pr.N) continue;
                    const float bias = pr.bias != nullptr ? load_as_float(pr.bias, P.bias_dtype, n) : 0.0f;
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        if (t >= P.M) break;
                        const float m = fused ? *(volatile const float*)(rs + t) : __ldg(rs + t);
                        const float f = apply_activation(fmaf(v[h][t] * pr.global_scale, m, bias), P.activation);
                        store_from_float(pr.out, P.out_dtype, static_cast<size_t>(t) * pr.ldo + n, f);
                    }
                }
            }
        }
    }

    if (warp == 2 && lane == 0) TL(6);
    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
    if (threadIdx.x == 0) TL(7);
}

// ------------------------------------------------------------------------------------------
// Activation pieces in the tiled image: one CTA per token row t < 16 (rows >= M are zeroed).
// Same arithmetic as nvfp4_quantize_pieces_kernel in nvfp4_gemm.cu.
// ------------------------------------------------------------------------------------------
struct QuantActs {
    int count;
    const void* x[TPB200_MAX_ACTS];
    int ldx[TPB200_MAX_ACTS];
    int K[TPB200_MAX_ACTS];
    uint8_t* image[TPB200_MAX_ACTS];
    float* row_scale[TPB200_MAX_ACTS];
};

__global__ void __launch_bounds__(256) quantize_pieces_tiled_kernel(const __grid_constant__ QuantActs A, int x_dtype,
                                                                    int M, int pieces) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int t = blockIdx.x;                 // 0..15
    const void* __restrict__ x = A.x[blockIdx.y];
    const int ldx = A.ldx[blockIdx.y];
    const int K = A.K[blockIdx.y];
    uint8_t* __restrict__ x_image = A.image[blockIdx.y];
    float* __restrict__ row_scale = A.row_scale[blockIdx.y];
    const int NB = 16 * pieces;
    const int nblk = K >> 4;
    const int kb_pad = (K + 255) / 256 * 16;
    __shared__ float red[8];
    float amax = 0.0f;
    if (t < M) {
        for (int kb = threadIdx.x; kb < nblk; kb += blockDim.x) {
            float r[16];
            load16_as_float(x, x_dtype, static_cast<size_t>(t) * ldx + kb * 16, r);
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(r[i]));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) amax = fmaxf(amax, red[i]);
    const int e = prescale_exponent(amax);
    const float pre = ldexpf(1.0f, e);
    if (threadIdx.x == 0 && t < M) row_scale[t] = ldexpf(1.0f, -e);

    for (int kb = threadIdx.x; kb < kb_pad; kb += blockDim.x) {
        float r[16];
        const bool valid = (t < M) && (kb < nblk);
        if (valid) {
            load16_as_float(x, x_dtype, static_cast<size_t>(t) * ldx + kb * 16, r);
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] *= pre;
        }
        const int ks = kb >> 4;
        const int c = (kb & 15) >> 1;            // 16-byte chunk of the 128-byte row
        for (int p = 0; p < pieces; ++p) {
            const int prow = p * 16 + t;
            uint8_t* blk = x_image + static_cast<size_t>(ks) * (NB * 128 + 2048);
            uint8_t* dst = blk + prow * 128 + ((c ^ (prow & 7)) << 4) + (kb & 1) * 8;
            uint8_t* sf_dst = blk + NB * 128 + ((kb >> 2) & 3) * 512 + (prow & 31) * 16 + ((prow >> 5) & 3) * 4 + (kb & 3);
            if (!valid) {
                *sf_dst = 0;
                *reinterpret_cast<uint2*>(dst) = make_uint2(0u, 0u);
                continue;
            }
            uint32_t lo, hi;
            *sf_dst = quantize_block16_piece(r, lo, hi);
            *reinterpret_cast<uint2*>(dst) = make_uint2(lo, hi);
        }
    }
}

}  // namespace

int device_error_gemv_tc(int clear) { return read_device_error(clear); }

}  // namespace tpb

// ---------------------------------------------------------------------------------------------
// Host side: the planner.  No heap: every table is a fixed-size member of a thread-local object, so
// the entry points allocate nothing, on the device or on the host.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kSmallUnits = 192;
constexpr int kLargeUnits = 1024;
constexpr int kMaxPieces = kLargeUnits;      // a candidate cut with more pieces than a launch can list is skipped

struct Shape {
    int N, K;
};

struct Piece {
    uint16_t p, rt, ks0, ks1;
    int16_t cta;
};
constexpr int16_t kPoolCta = 0x7FFF;         // sorts after every CTA

struct Plan {
    tpb::TcUnit units[kLargeUnits];          // CTA by CTA
    uint16_t cta_begin[tpb::kMaxCtas + 1];
    int num_units = 0;
    int grid = 0;
    int pool_begin = 0, pool_size = 0;       // units[pool_begin ...) are not tied to a CTA
    size_t slots = 0;                        // partial-sum slots (16 * 256 floats each)
    size_t counters = 0;                     // arrival counters of cut tiles; the pool's ticket counter follows them
    int max_load = 0;                        // stages of the longest CTA's fixed list
};

struct PlanScratch {
    Piece pieces[kMaxPieces];
    Piece best[kMaxPieces];
    int num = 0, num_best = 0, grid_best = 0;
    int load[tpb::kMaxCtas];
    int heap[tpb::kMaxCtas];                 // CTA ids ordered by load (binary min-heap)
    int order[kLargeUnits];
};

// Deal the pieces of one candidate cut (no piece longer than `lmax` stages) to the CTAs, longest first,
// each to the least loaded CTA; returns the largest load in stages, or -1 if the cut has too many pieces.
int deal(const Shape* shapes, int count, int sms, int lmax, PlanScratch& S, bool& any_cut) {
    S.num = 0;
    any_cut = false;
    for (int p = 0; p < count; ++p) {
        const int row_tiles = (shapes[p].N + 255) / 256;
        const int k_stages = (shapes[p].K + 255) / 256;
        const int cuts = (k_stages + lmax - 1) / lmax;
        const int len = (k_stages + cuts - 1) / cuts;
        if (cuts > 1) any_cut = true;
        for (int rt = 0; rt < row_tiles; ++rt) {
            for (int k0 = 0; k0 < k_stages; k0 += len) {
                if (S.num == kMaxPieces) return -1;
                S.pieces[S.num++] = {static_cast<uint16_t>(p), static_cast<uint16_t>(rt), static_cast<uint16_t>(k0),
                                     static_cast<uint16_t>(std::min(k_stages, k0 + len)), 0};
            }
        }
    }
    // longest first; ties in launch order (a total order, so std::sort is deterministic)
    std::sort(S.pieces, S.pieces + S.num, [](const Piece& a, const Piece& b) {
        const int la = a.ks1 - a.ks0, lb = b.ks1 - b.ks0;
        if (la != lb) return la > lb;
        if (a.p != b.p) return a.p < b.p;
        if (a.rt != b.rt) return a.rt < b.rt;
        return a.ks0 < b.ks0;
    });
    const int grid = std::min(sms, S.num);
    for (int c = 0; c < grid; ++c) {
        S.load[c] = 0;
        S.heap[c] = c;
    }
    auto heavier = [&S](int a, int b) { return S.load[a] != S.load[b] ? S.load[a] > S.load[b] : a > b; };
    for (int i = 0; i < S.num; ++i) {
        std::pop_heap(S.heap, S.heap + grid, heavier);           // least loaded CTA moves to the back
        const int c = S.heap[grid - 1];
        S.pieces[i].cta = static_cast<int16_t>(c);
        S.load[c] += S.pieces[i].ks1 - S.pieces[i].ks0;
        std::push_heap(S.heap, S.heap + grid, heavier);
    }
    return *std::max_element(S.load, S.load + grid);
}

// Candidate cuts: tiles whole, or no piece longer than 16 / 8 / 4 / 2 / 1 stages.  A cut costs a hand-over of
// partial sums through global memory at the end of the launch (about five stage times, plus the last
// arriver's walk over the tile's pieces), so it is taken only when it shortens the longest CTA by more.
int make_plan(const Shape* shapes, int count, int sms, Plan& plan, PlanScratch& S) {
    if (sms < 1 || sms > tpb::kMaxCtas) return TPB200_ERR_CUDA;
    int longest = 1;
    for (int i = 0; i < count; ++i) {
        const Shape& s = shapes[i];
        if (s.N < 1 || s.K < 16 || s.K % 16 != 0) return TPB200_ERR_SHAPE;
        if ((s.N + 255) / 256 > 65535 || (s.K + 255) / 256 > 65535) return TPB200_ERR_SHAPE;
        longest = std::max(longest, (s.K + 255) / 256);
    }
    constexpr int kHandOverStages = 5;
    constexpr int kWhole = 1 << 30;
    int best_cost = 0;
    bool have = false;
    for (int lmax : {kWhole, 16, 8, 4, 2, 1}) {
        if (lmax != kWhole && lmax >= longest) continue;           // same as the whole-tile plan
        bool any_cut = false;
        const int load = deal(shapes, count, sms, lmax, S, any_cut);
        if (load < 0) continue;
        int cost = load;
        if (any_cut) {
            int max_cuts = 1;
            for (int i = 0; i < count; ++i) {
                const int ks = (shapes[i].K + 255) / 256;
                max_cuts = std::max(max_cuts, (ks + lmax - 1) / lmax);
            }
            cost += kHandOverStages + max_cuts / 8;
        }
        if (!have || cost < best_cost) {
            std::copy(S.pieces, S.pieces + S.num, S.best);
            S.num_best = S.num;
            S.grid_best = std::min(sms, S.num);
            best_cost = cost;
            have = true;
        }
    }
    if (!have) return TPB200_ERR_SHAPE;                            // more tiles than one launch can list
    // A launch that fills the machine several times over ties only ONE unit to each CTA (the smallest ones:
    // they are what the CTAs request before griddepcontrol.wait) and leaves the rest in the pool, longest
    // first.  SMs do not get equal shares of the memory system -- a CTA can need 40 % longer per stage than
    // its neighbour -- and a long unit tied to a slow CTA would be the last thing the launch waits for.
    if (S.grid_best == sms && S.num_best >= 2 * sms) {
        for (int i = 0; i < S.num_best; ++i) {
            const int from_end = S.num_best - 1 - i;               // the list is sorted longest first
            S.best[i].cta = from_end < sms ? static_cast<int16_t>(from_end) : kPoolCta;
        }
    }

    // CTA by CTA: whole tiles first, cut tiles last (their hand-over then holds up nothing that follows);
    // neighbouring pieces of one tile that landed on the same CTA become one unit.
    auto k_stages = [&](int p) { return (shapes[p].K + 255) / 256; };
    std::sort(S.best, S.best + S.num_best, [&](const Piece& a, const Piece& b) {
        if (a.cta != b.cta) return a.cta < b.cta;
        if (a.cta == kPoolCta && (a.ks1 - a.ks0) != (b.ks1 - b.ks0)) return (a.ks1 - a.ks0) > (b.ks1 - b.ks0);
        const bool ca = (a.ks1 - a.ks0) != k_stages(a.p), cb = (b.ks1 - b.ks0) != k_stages(b.p);
        if (ca != cb) return !ca;
        if (a.p != b.p) return a.p < b.p;
        if (a.rt != b.rt) return a.rt < b.rt;
        return a.ks0 < b.ks0;
    });
    plan.num_units = 0;
    plan.grid = S.grid_best;
    plan.max_load = 0;
    int i = 0;
    for (int c = 0; c < plan.grid; ++c) {
        plan.cta_begin[c] = static_cast<uint16_t>(plan.num_units);
        const int first = plan.num_units;
        int load = 0;
        for (; i < S.num_best && S.best[i].cta == c; ++i) {
            const Piece& pc = S.best[i];
            load += pc.ks1 - pc.ks0;
            if (plan.num_units > first) {
                tpb::TcUnit& last = plan.units[plan.num_units - 1];
                if (last.p == pc.p && last.rt == pc.rt && last.ks1 == pc.ks0) {
                    last.ks1 = pc.ks1;
                    continue;
                }
            }
            if (plan.num_units == kLargeUnits) return TPB200_ERR_SHAPE;
            tpb::TcUnit u = {};
            u.p = static_cast<uint8_t>(pc.p);
            u.rt = pc.rt;
            u.ks0 = pc.ks0;
            u.ks1 = pc.ks1;
            plan.units[plan.num_units++] = u;
        }
        plan.max_load = std::max(plan.max_load, load);
    }
    plan.cta_begin[plan.grid] = static_cast<uint16_t>(plan.num_units);
    plan.pool_begin = plan.num_units;
    for (; i < S.num_best; ++i) {                                  // the pool, longest first, nothing merged
        const Piece& pc = S.best[i];
        if (plan.num_units == kLargeUnits) return TPB200_ERR_SHAPE;
        tpb::TcUnit u = {};
        u.p = static_cast<uint8_t>(pc.p);
        u.rt = pc.rt;
        u.ks0 = pc.ks0;
        u.ks1 = pc.ks1;
        plan.units[plan.num_units++] = u;
    }
    plan.pool_size = plan.num_units - plan.pool_begin;
    // cut tiles: slots in K order, one counter per tile
    int ncut = 0;
    for (int k = 0; k < plan.num_units; ++k) {
        const tpb::TcUnit& u = plan.units[k];
        if (u.ks1 - u.ks0 != k_stages(u.p)) S.order[ncut++] = k;
    }
    std::sort(S.order, S.order + ncut, [&](int a, int b) {
        const tpb::TcUnit &x = plan.units[a], &y = plan.units[b];
        if (x.p != y.p) return x.p < y.p;
        if (x.rt != y.rt) return x.rt < y.rt;
        return x.ks0 < y.ks0;
    });
    plan.slots = 0;
    plan.counters = 0;
    for (int a = 0; a < ncut;) {
        int b = a;
        while (b < ncut && plan.units[S.order[b]].p == plan.units[S.order[a]].p &&
               plan.units[S.order[b]].rt == plan.units[S.order[a]].rt) {
            ++b;
        }
        const int n = b - a;
        if (n > 255 || plan.slots + n > 65535 || plan.counters > 65535) return TPB200_ERR_SHAPE;
        for (int k = a; k < b; ++k) {
            tpb::TcUnit& u = plan.units[S.order[k]];
            u.shared = 1;
            u.slot0 = static_cast<uint16_t>(plan.slots);
            u.counter = static_cast<uint16_t>(plan.counters);
            u.slot = static_cast<uint8_t>(k - a);
            u.nslots = static_cast<uint8_t>(n);
        }
        plan.slots += n;
        plan.counters += 1;
        a = b;
    }
    return TPB200_OK;
}

int device_sms(int& sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    return TPB200_OK;
}

// arrival counters of the cut tiles, then the pool's ticket counter
size_t counter_bytes(const Plan& plan) { return ((plan.counters + 1) * sizeof(int) + 255) / 256 * 256; }
bool needs_workspace(const Plan& plan) { return plan.slots > 0 || plan.pool_size > 0; }
size_t workspace_bytes(const Plan& plan) {
    return needs_workspace(plan) ? counter_bytes(plan) + plan.slots * tpb::kSlotFloats * sizeof(float) : 0;
}

// Plans are remembered per calling thread for the last few distinct shape lists: a decode loop launches
// the same handful of groups over and over.
struct PlanCache {
    static constexpr int kEntries = 8;
    struct Entry {
        int count = 0, sms = 0;
        Shape shapes[TPB200_MAX_GROUP];
        Plan plan;
    };
    Entry entries[kEntries];
    int next = 0;
    PlanScratch scratch;

    int get(const Shape* shapes, int count, const Plan** out) {
        int sms = 0;
        if (device_sms(sms) != TPB200_OK) return TPB200_ERR_CUDA;
        for (Entry& e : entries) {
            if (e.count == count && e.sms == sms &&
                std::equal(shapes, shapes + count, e.shapes, [](const Shape& a, const Shape& b) { return a.N == b.N && a.K == b.K; })) {
                *out = &e.plan;
                return TPB200_OK;
            }
        }
        Entry& e = entries[next];
        e.count = 0;                                 // invalid while it is rebuilt
        const int st = make_plan(shapes, count, sms, e.plan, scratch);
        if (st != TPB200_OK) return st;
        std::copy(shapes, shapes + count, e.shapes);
        e.count = count;
        e.sms = sms;
        next = (next + 1) % kEntries;
        *out = &e.plan;
        return TPB200_OK;
    }
};

PlanCache& plan_cache() {
    static thread_local PlanCache cache;
    return cache;
}

// Everything a launch needs, validated and planned on the host BEFORE anything is enqueued.
struct Launch {
    Shape shapes[TPB200_MAX_GROUP];
    tpb::TcProblem prob[TPB200_MAX_GROUP];
    int count = 0;
    const Plan* plan = nullptr;
    int M = 0, pieces = 0, x_dtype = TPB200_BF16, bias_dtype = TPB200_F32, out_dtype = TPB200_BF16, activation = 0;
    int fused = 0, flags = 0;
};

int check_common(int count, int M, int pieces, int bias_dtype, int out_dtype, int activation, int flags) {
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_GROUP, TPB200_ERR_SHAPE);
    TPB_REQUIRE(M >= 1 && M <= 16 && pieces >= 1 && pieces <= 4, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(bias_dtype) && tpb_valid_dtype(out_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE(activation >= TPB200_ACT_NONE && activation <= TPB200_ACT_SILU, TPB200_ERR_ENUM);
    TPB_REQUIRE((flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    return TPB200_OK;
}

template <int kMaxUnits>
int launch_with(const Launch& L, void* workspace, tpb200_stream_t stream) {
    static thread_local tpb::TcParams<kMaxUnits> P;      // ~8 / ~21 KB: kept off the caller's stack
    const Plan& plan = *L.plan;
    P.num_problems = L.count;
    P.M = L.M;
    P.pieces = L.pieces;
    P.x_dtype = L.x_dtype;
    P.bias_dtype = L.bias_dtype;
    P.out_dtype = L.out_dtype;
    P.activation = L.activation;
    P.fused = L.fused;
    static std::atomic<int> launch_number{0};
    P.debug_slot = launch_number.fetch_add(1, std::memory_order_relaxed);
    P.counters = static_cast<int*>(workspace);
    P.queue = reinterpret_cast<unsigned int*>(workspace) + plan.counters;
    P.pool_begin = plan.pool_begin;
    P.pool_size = plan.pool_size;
    P.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counter_bytes(plan));
    std::copy(L.prob, L.prob + L.count, P.prob);
    std::copy(plan.cta_begin, plan.cta_begin + plan.grid + 1, P.cta_begin);
    std::copy(plan.units, plan.units + plan.num_units, P.units);

    const size_t smem = tpb::num_stages(L.pieces) * tpb::stage_bytes(L.pieces) + sizeof(tpb::SharedControl) + 1024;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(tpb::nvfp4_gemv_tc_kernel<kMaxUnits>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid, 1, 1);
    cfg.blockDim = dim3(tpb::kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (L.flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, tpb::nvfp4_gemv_tc_kernel<kMaxUnits>, P) != cudaSuccess) return TPB200_ERR_CUDA;
    return TPB200_OK;
}

int launch(const Launch& L, void* workspace, size_t workspace_size, tpb200_stream_t stream) {
    if (needs_workspace(*L.plan)) {
        TPB_REQUIRE(workspace != nullptr, TPB200_ERR_WORKSPACE);
        TPB_REQUIRE(workspace_size >= workspace_bytes(*L.plan), TPB200_ERR_WORKSPACE);
        TPB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, TPB200_ERR_ALIGN);
    }
    if (L.plan->num_units <= kSmallUnits) return launch_with<kSmallUnits>(L, workspace, stream);
    return launch_with<kLargeUnits>(L, workspace, stream);
}

Launch& launch_record() {
    static thread_local Launch L;
    return L;
}

int prepare_pretiled(const tpb200_gemv_tc_problem* problems, int count, int M, int pieces, int bias_dtype, int out_dtype,
                     int activation, int flags, Launch& L) {
    TPB_REQUIRE(problems != nullptr, TPB200_ERR_NULL);
    const int st = check_common(count, M, pieces, bias_dtype, out_dtype, activation, flags);
    if (st != TPB200_OK) return st;
    L.count = count;
    L.M = M;
    L.pieces = pieces;
    L.x_dtype = TPB200_BF16;
    L.bias_dtype = bias_dtype;
    L.out_dtype = out_dtype;
    L.activation = activation;
    L.flags = flags;
    L.fused = 0;
    for (int i = 0; i < count; ++i) {
        const tpb200_gemv_tc_problem& h = problems[i];
        TPB_REQUIRE(h.w_image && h.x_image && h.x_row_scale && h.out, TPB200_ERR_NULL);
        TPB_REQUIRE(tpb_aligned16(h.w_image) && tpb_aligned16(h.x_image), TPB200_ERR_ALIGN);
        TPB_REQUIRE(h.ldo == 0 || h.ldo >= h.N, TPB200_ERR_SHAPE);
        tpb::TcProblem d = {};
        d.w_image = static_cast<const uint8_t*>(h.w_image);
        d.x = h.x_image;
        d.row_scale = h.x_row_scale;
        d.bias = h.bias;
        d.out = h.out;
        d.N = h.N;
        d.K = h.K;
        d.ldo = h.ldo == 0 ? h.N : h.ldo;
        d.ldx = 0;
        d.global_scale = h.global_scale;
        d.k_stages = (h.K + 255) / 256;
        L.prob[i] = d;
        L.shapes[i] = {h.N, h.K};
    }
    return plan_cache().get(L.shapes, count, &L.plan);
}

int prepare_fused(const tpb200_gemv_tc_fused_problem* problems, int count, int M, int pieces, int x_dtype, int bias_dtype,
                  int out_dtype, int activation, int flags, Launch& L) {
    TPB_REQUIRE(problems != nullptr, TPB200_ERR_NULL);
    const int st = check_common(count, M, pieces, bias_dtype, out_dtype, activation, flags);
    if (st != TPB200_OK) return st;
    TPB_REQUIRE(tpb_valid_dtype(x_dtype), TPB200_ERR_ENUM);
    L.count = count;
    L.M = M;
    L.pieces = pieces;
    L.x_dtype = x_dtype;
    L.bias_dtype = bias_dtype;
    L.out_dtype = out_dtype;
    L.activation = activation;
    L.flags = flags;
    L.fused = 1;
    for (int i = 0; i < count; ++i) {
        const tpb200_gemv_tc_fused_problem& h = problems[i];
        TPB_REQUIRE(h.w_image && h.x && h.out, TPB200_ERR_NULL);
        TPB_REQUIRE(tpb_aligned16(h.w_image) && tpb_aligned16(h.x), TPB200_ERR_ALIGN);
        TPB_REQUIRE(h.ldo == 0 || h.ldo >= h.N, TPB200_ERR_SHAPE);
        const int ldx = h.ldx == 0 ? h.K : h.ldx;
        TPB_REQUIRE(ldx >= h.K, TPB200_ERR_SHAPE);
        TPB_REQUIRE((static_cast<long long>(ldx) * tpb_dtype_size(x_dtype)) % 16 == 0, TPB200_ERR_ALIGN);
        tpb::TcProblem d = {};
        d.w_image = static_cast<const uint8_t*>(h.w_image);
        d.x = h.x;
        d.row_scale = nullptr;
        d.bias = h.bias;
        d.out = h.out;
        d.N = h.N;
        d.K = h.K;
        d.ldo = h.ldo == 0 ? h.N : h.ldo;
        d.ldx = ldx;
        d.global_scale = h.global_scale;
        d.k_stages = (h.K + 255) / 256;
        L.prob[i] = d;
        L.shapes[i] = {h.N, h.K};
    }
    return plan_cache().get(L.shapes, count, &L.plan);
}

size_t planned_workspace(const Shape* shapes, int count) {
    const Plan* plan = nullptr;
    if (plan_cache().get(shapes, count, &plan) != TPB200_OK) return 0;
    // counters first (zero-initialised by the caller once), then the partial sums
    return workspace_bytes(*plan) + 256;
}

}  // namespace

extern "C" size_t tpb200_nvfp4_gemv_tc_workspace_size(const tpb200_gemv_tc_problem* problems, int count) {
    if (problems == nullptr || count < 1 || count > TPB200_MAX_GROUP) return 0;
    Shape shapes[TPB200_MAX_GROUP];
    for (int i = 0; i < count; ++i) shapes[i] = {problems[i].N, problems[i].K};
    return planned_workspace(shapes, count);
}

extern "C" size_t tpb200_nvfp4_gemv_tc_fused_workspace_size(const tpb200_gemv_tc_fused_problem* problems, int count) {
    if (problems == nullptr || count < 1 || count > TPB200_MAX_GROUP) return 0;
    Shape shapes[TPB200_MAX_GROUP];
    for (int i = 0; i < count; ++i) shapes[i] = {problems[i].N, problems[i].K};
    return planned_workspace(shapes, count);
}

extern "C" int tpb200_nvfp4_gemv_tc_plan(const int* N, const int* K, int count, int sms, tpb200_gemv_tc_plan_info* info) {
    TPB_REQUIRE(N && K && info, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_GROUP, TPB200_ERR_SHAPE);
    TPB_REQUIRE(sms >= 1 && sms <= tpb::kMaxCtas, TPB200_ERR_SHAPE);
    static thread_local Plan plan;
    static thread_local PlanScratch scratch;
    Shape shapes[TPB200_MAX_GROUP];
    long long total = 0;
    for (int i = 0; i < count; ++i) {
        shapes[i] = {N[i], K[i]};
        total += static_cast<long long>((N[i] + 255) / 256) * ((K[i] + 255) / 256);
    }
    const int st = make_plan(shapes, count, sms, plan, scratch);
    if (st != TPB200_OK) return st;
    info->grid = plan.grid;
    info->units = plan.num_units;
    info->max_load_stages = plan.max_load;
    info->total_stages = static_cast<int>(total);
    info->cut_tiles = static_cast<int>(plan.counters);
    info->pool_units = plan.pool_size;
    info->workspace_bytes = workspace_bytes(plan);
    return TPB200_OK;
}

#ifdef TPB_TIMELINE
// Diagnostic build only: copies the stamps of the last kTlSlots launches ([slot][CTA][point], nanoseconds)
// and returns the launch number the next launch will get.
extern "C" int tpb200_debug_gemv_tc_timeline(unsigned long long* out, size_t bytes) {
    if (bytes > sizeof(tpb::g_timeline)) bytes = sizeof(tpb::g_timeline);
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out, tpb::g_timeline, bytes);
    return 0;
}
#endif

extern "C" size_t tpb200_nvfp4_gemv_tc_x_image_bytes(int K, int pieces) {
    if (K < 16 || pieces < 1 || pieces > 4) return 0;
    return static_cast<size_t>((K + 255) / 256) * (16 * pieces * 128 + 2048);
}

extern "C" int tpb200_nvfp4_quantize_acts_tc(const tpb200_act_tc* acts, int count, int x_dtype, int M, int pieces,
                                             int flags, tpb200_stream_t stream) {
    TPB_REQUIRE(acts != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_ACTS, TPB200_ERR_SHAPE);
    TPB_REQUIRE(M >= 1 && M <= 16 && pieces >= 1 && pieces <= 4, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(x_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE((flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    tpb::QuantActs A;
    A.count = count;
    for (int i = 0; i < count; ++i) {
        const tpb200_act_tc& h = acts[i];
        TPB_REQUIRE(h.x && h.x_image && h.x_row_scale, TPB200_ERR_NULL);
        TPB_REQUIRE(h.K >= 16 && h.K % 16 == 0 && h.ldx >= h.K, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(h.x) && tpb_aligned16(h.x_image), TPB200_ERR_ALIGN);
        TPB_REQUIRE((static_cast<long long>(h.ldx) * tpb_dtype_size(x_dtype)) % 16 == 0, TPB200_ERR_ALIGN);
        A.x[i] = h.x;
        A.ldx[i] = h.ldx;
        A.K[i] = h.K;
        A.image[i] = static_cast<uint8_t*>(h.x_image);
        A.row_scale[i] = h.x_row_scale;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16, count, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, tpb::quantize_pieces_tiled_kernel, A, x_dtype, M, pieces) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    return TPB200_OK;
}

extern "C" int tpb200_nvfp4_quantize_act_tc(const void* x, int x_dtype, int ldx, void* x_image, float* row_scale, int M,
                                            int K, int pieces, int flags, tpb200_stream_t stream) {
    tpb200_act_tc a = {x, ldx, K, x_image, row_scale};
    return tpb200_nvfp4_quantize_acts_tc(&a, 1, x_dtype, M, pieces, flags, stream);
}

extern "C" int tpb200_nvfp4_gemv_tc(const tpb200_gemv_tc_problem* problems, int count, int M, int pieces,
                                    int bias_dtype, int out_dtype, int activation, void* workspace,
                                    size_t workspace_size, int flags, tpb200_stream_t stream) {
    Launch& L = launch_record();
    const int st = prepare_pretiled(problems, count, M, pieces, bias_dtype, out_dtype, activation, flags, L);
    if (st != TPB200_OK) return st;
    return launch(L, workspace, workspace_size, stream);
}

extern "C" int tpb200_nvfp4_gemv_tc_fused(const tpb200_gemv_tc_fused_problem* problems, int count, int M, int pieces,
                                          int x_dtype, int bias_dtype, int out_dtype, int activation, void* workspace,
                                          size_t workspace_size, int flags, tpb200_stream_t stream) {
    Launch& L = launch_record();
    const int st = prepare_fused(problems, count, M, pieces, x_dtype, bias_dtype, out_dtype, activation, flags, L);
    if (st != TPB200_OK) return st;
    return launch(L, workspace, workspace_size, stream);
}

// ---------------------------------------------------------------------------------------------
// The same GEMV for callers that are not able to allocate device memory.
//
// tpb200_nvfp4_gemv_tc needs a workspace for the partial sums and arrival counters of tiles that its
// plan cuts along K.  Some callers have nowhere to get one from: a TensorRT plugin whose enqueue() was
// not granted a workspace, a robot-control loop that must not touch the allocator once it is running,
// host code that is handed raw pointers and no allocator of the framework that owns them.  For them the
// scratch lives in the library image itself, in the array below.  Every GPU that loads the library
// carries these 4 MiB until the process exits.
//
// Host code must not hand `g_static_scratch` to a kernel directly: in host code that name is only a
// stand-in for the symbol, not a device address.  The address is looked up once per device with
// cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// device-side address of g_static_scratch per device ordinal, filled on first use
std::atomic<void*> g_static_scratch_addr[64];

int static_scratch_address(void** out) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB200_ERR_CUDA;
    void* p = g_static_scratch_addr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return TPB200_ERR_CUDA;
        g_static_scratch_addr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return TPB200_OK;
}

}  // namespace

extern "C" size_t tpb200_nvfp4_gemv_tc_static_capacity(void) { return kStaticScratchBytes; }

extern "C" int tpb200_nvfp4_gemv_tc_static(const tpb200_gemv_tc_problem* problems, int count, int M, int pieces,
                                           int bias_dtype, int out_dtype, int activation, int flags,
                                           tpb200_stream_t stream) {
    // every argument is validated and the launch planned before anything is enqueued
    Launch& L = launch_record();
    const int st = prepare_pretiled(problems, count, M, pieces, bias_dtype, out_dtype, activation, flags, L);
    if (st != TPB200_OK) return st;
    // larger plans than the built-in scratch can hold are refused, never truncated
    TPB_REQUIRE(workspace_bytes(*L.plan) <= kStaticScratchBytes, TPB200_ERR_WORKSPACE);
    void* scratch = nullptr;
    const int sa = static_scratch_address(&scratch);
    if (sa != TPB200_OK) return sa;
    // The array keeps whatever the previous call left.  Only the tile counters have to start at
    // zero; the partial sums are always written before they are read.
    const size_t cb = needs_workspace(*L.plan) ? counter_bytes(*L.plan) : 0;
    if (cb > 0 && cudaMemsetAsync(scratch, 0, cb, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    return launch(L, scratch, kStaticScratchBytes, stream);
}
