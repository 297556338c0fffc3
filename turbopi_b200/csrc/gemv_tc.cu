// Decode-shaped (M <= 16 tokens) NVFP4 weight-only GEMV on the tensor cores.
//
// The CUDA-core GEMV is bound by instruction issue (decode + FMA per weight); here the SM does
// no per-weight work at all.  The roles of a GEMM are swapped: a 128-row slab of the WEIGHT
// matrix is the A operand of tcgen05.mma kind::mxf4nvf4, the activations are the B operand.
// bf16 activations keep their precision as residual e2m1 pieces (see nvfp4_gemm.cu) stacked
// along N: piece p of token t is B row 16 p + t, so one MMA (N = 16 * pieces) per 64-wide K
// atom handles all pieces and the epilogue adds the pieces' columns.
//
// Both operands are stored PRE-TILED in the shared-memory image of the 128-byte swizzle, scales
// included, so that a stage is TWO plain 1-D bulk copies -- no tensor maps, any number of problems
// per launch:
//   weights      the tensor-core GEMM's B image (tpb200_nvfp4_tile_weights): block (n_blk, ks) of
//                36 KB = 256 rows x 128 B of codes (16-byte chunk c of row r at c ^ (r & 7)) + the two
//                2 KB scale slabs; one image serves the prefill GEMM and this decode GEMV;
//   activations  block ks = 16 * pieces rows x 128 B of codes in the same pattern + one 2 KB scale slab.
// A stage (36 KB of weights + <= 10 KB of activations) feeds two MMAs per 64-wide K atom (weight rows
// 0..127 and 128..255, two accumulators) against the same activation operand.
//
// One lane issues the two bulk copies of a stage; a ring of four stages (176 KB) keeps the stream
// going.  (Streaming alone is not the limit: a ring of 36-48 KB bulk copies reads HBM at 7.1 TB/s
// over 148 SMs when nothing consumes the data, and four warps of 16-byte cp.async copies do no
// better.  What this kernel adds per stage -- scale copies and MMAs between `full` and `empty`,
// and the fenced hand-over of split-K partial sums -- is what keeps it at ~3 TB/s.)
//
// Work unit = (problem, 256-row tile, K split); all units carry (nearly) the same number of stages
// and every CTA owns a contiguous range of equally many.  Consecutive units of one tile inside a
// CTA's range form a GROUP that is accumulated in tensor memory as one K range, so only the tiles cut
// by a range boundary are shared between CTAs: each of their groups writes its partial sums (only the
// valid tokens) to caller-provided scratch, and the CTA that arrives last on the tile's counter adds
// them in K order (deterministic), applies the epilogue and resets the counter.  Nothing ever waits
// on another CTA.  (Handing over partial sums costs a device-wide fence, ~2.5 us per hand-over; with
// one per unit the CTAs that drew down-projection units finished 17 us after the others.)
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
    return (227 * 1024 - 2048) / stage_bytes(pieces) < kMaxStages ? (227 * 1024 - 2048) / stage_bytes(pieces) : kMaxStages;
}
constexpr int kThreads = 224;          // warps: 0 producer, 1 MMA issuer, 2..5 epilogue, 6 scale copier
constexpr int kTmemCols = 512;
// tensor memory: accumulator (buffer b, row half h) at column b * 128 + h * 64, then the scales
// two sets of scale columns (stages alternate): 32 for the weights' two row halves + 16 for the activations
constexpr uint32_t kSfSetCols = 48;
constexpr uint32_t kSfaCol = 256;
constexpr uint32_t kSfbCol = kSfaCol + 32;
constexpr int kMaxProblems = TPB200_MAX_GROUP;

struct TcProblem {
    const uint8_t* w_image;     // [row_tiles of 256][k_stages][36864]
    const uint8_t* x_image;     // [k_stages][NB * 128 + 2048]
    const float* row_scale;     // [M]
    const void* bias;
    void* out;
    int N, K;
    int ldo;
    float global_scale;
    int k_stages;
    int row_tiles;
    int splits;                 // K splits per row tile
    int stages_per_split;
    int unit_begin;
    int scratch_off;            // float offset of this problem's partials [splits][16][row_tiles*128]
    int counter_off;            // int offset of this problem's per-tile counters
};

struct TcParams {
    int num_problems;
    int total_units;
    int M;
    int pieces;
    int bias_dtype, out_dtype, activation;
    float* scratch;
    int* counters;
    TcProblem prob[kMaxProblems];
};

struct SharedControl {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t sf_full[2];      // scale set j copied into tensor memory (arrives through tcgen05.commit)
    uint64_t sf_empty[2];     // the MMAs that read scale set j are done
    uint32_t tmem_base;
    int abort_flag;
    int ticket;
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

struct Unit {
    int p, rt, split, ks0, ks1;
};

// Index of the problem that owns unit u, by bisection.  The problem table sits in the kernel's parameter
// space and every dependent look-up with a computed index costs ~100 cycles; walking the table from its
// start made the CTAs of the last problems begin their work 8 us after the first ones.
__device__ __forceinline__ int find_problem(const TcParams& P, int u) {
    int lo = 0, hi = P.num_problems - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (u >= P.prob[mid].unit_begin) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

__device__ __forceinline__ Unit decode_unit(const TcParams& P, int u, int& p_hint) {
    while (p_hint + 1 < P.num_problems && u >= P.prob[p_hint + 1].unit_begin) ++p_hint;
    const TcProblem& pr = P.prob[p_hint];
    const int local = u - pr.unit_begin;
    Unit un;
    un.p = p_hint;
    un.rt = local / pr.splits;
    un.split = local - un.rt * pr.splits;
    un.ks0 = un.split * pr.stages_per_split;
    un.ks1 = min(pr.k_stages, un.ks0 + pr.stages_per_split);
    return un;
}

// The group that starts at unit u: the units of u's tile from u to the end of the tile or of the CTA's range.
struct Group {
    int p, rt, split0, split1, ks0, ks1, next;
};

__device__ __forceinline__ Group decode_group(const TcParams& P, int u, int unit_hi, int& p_hint) {
    const Unit un = decode_unit(P, u, p_hint);
    const TcProblem& pr = P.prob[un.p];
    const int tile_end = pr.unit_begin + (un.rt + 1) * pr.splits;
    Group g;
    g.p = un.p;
    g.rt = un.rt;
    g.split0 = un.split;
    g.next = min(unit_hi, tile_end);
    g.split1 = un.split + (g.next - u) - 1;
    g.ks0 = un.ks0;
    g.ks1 = min(pr.k_stages, (g.split1 + 1) * pr.stages_per_split);
    return g;
}

__global__ void __launch_bounds__(kThreads, 1) nvfp4_gemv_tc_kernel(const __grid_constant__ TcParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int kStages = num_stages(P.pieces);
    const int kStageBytes = stage_bytes(P.pieces);
    SharedControl* ctl = reinterpret_cast<SharedControl*>(smem + kStages * kStageBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int NB = 16 * P.pieces;
    const int unit_lo = static_cast<int>(static_cast<long long>(blockIdx.x) * P.total_units / gridDim.x);
    const int unit_hi = static_cast<int>(static_cast<long long>(blockIdx.x + 1) * P.total_units / gridDim.x);
    const int p_first = find_problem(P, unit_lo);     // every role starts its table walk here

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);
            mbar_init(&ctl->sf_full[b], 1);
            mbar_init(&ctl->sf_empty[b], 1);
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
    pdl_launch_dependents();

    if (warp == 0) {
        // ------------------------------------------------------------ producer (whole warp): lane 0 owns the
        // barrier hand-shakes, lanes 0..3 each copy a quarter of the stage's weight block and lane 4 the
        // activation block.  (A thread that issues a bulk copy is held for ~0.3 us whatever the size; requests
        // issued side by side from several lanes overlap that.)  Weights never depend on the previous kernel,
        // so the first stages' weight blocks are requested before griddepcontrol.wait; the activation image
        // is written by the previous kernel.
        const uint32_t xbytes = static_cast<uint32_t>(NB) * 128u + kSfSlab;
        constexpr uint32_t kQuarter = kWBlock / 4;
        int pre = 0;
        {
            int ph = p_first;
            for (int u = unit_lo; u < unit_hi && pre < kStages; ++u) {
                const Unit un = decode_unit(P, u, ph);
                const TcProblem& pr = P.prob[un.p];
                for (int ks = un.ks0; ks < un.ks1 && pre < kStages; ++ks, ++pre) {
                    uint8_t* st = smem + pre * kStageBytes;
                    const size_t blk = static_cast<size_t>(un.rt) * pr.k_stages + ks;
                    if (lane == 0) mbar_expect_tx(&ctl->full[pre], kWBlock + xbytes);
                    __syncwarp();
                    if (lane < 4) {
                        bulk_copy_g2s(st + lane * kQuarter, pr.w_image + blk * kWBlock + lane * kQuarter, kQuarter,
                                      &ctl->full[pre]);
                    }
                }
            }
        }
        pdl_wait_prior_grids();
        int it = 0, ph = p_first;
        bool stop = false;
        for (int u = unit_lo; u < unit_hi && !stop; ++u) {
            const Unit un = decode_unit(P, u, ph);
            const TcProblem& pr = P.prob[un.p];
            for (int ks = un.ks0; ks < un.ks1; ++ks, ++it) {
                const int s = it % kStages;
                uint8_t* st = smem + s * kStageBytes;
                const size_t blk = static_cast<size_t>(un.rt) * pr.k_stages + ks;
                int bad = 0;
                if (lane == 0) {
                    if (*abort_flag) {
                        bad = 1;
                    } else if (it >= pre) {
                        if (it >= kStages && !mbar_wait_bounded(&ctl->empty[s], ((it / kStages) - 1) & 1)) {
                            record_error(kErrGemmEmptyBarrierTimeout);
                            *abort_flag = 1;
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
                        bulk_copy_g2s(st + lane * kQuarter, pr.w_image + blk * kWBlock + lane * kQuarter, kQuarter,
                                      &ctl->full[s]);
                    }
                } else if (lane == 4) {
                    bulk_copy_g2s(st + kWBlock, pr.x_image + static_cast<size_t>(ks) * xbytes, xbytes, &ctl->full[s]);
                }
            }
        }
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
            int unit_iter = 0, ph = p_first;
            for (int u = unit_lo; u < unit_hi && !*abort_flag; ++unit_iter) {
                const Group un = decode_group(P, u, unit_hi, ph);
                u = un.next;
                const int buf = unit_iter & 1;
                if (unit_iter >= 2 && !mbar_wait_bounded(&ctl->acc_empty[buf], ((unit_iter >> 1) - 1) & 1)) {
                    record_error(kErrGemmEpilogueBarrierTimeout);
                    *abort_flag = 1;
                    break;
                }
                tc::fence_after_thread_sync();
                const uint32_t tmem_acc = tmem_base + buf * 128;
                uint32_t accumulate = 0;
                for (int ks = un.ks0; ks < un.ks1; ++ks) {
                    if (!mbar_wait_bounded(&ctl->full[s], full_phase)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    // the scale copier (warp 6) has moved this stage's scales into set g & 1
                    const uint32_t set = g & 1u;
                    if (!mbar_wait_bounded(&ctl->sf_full[set], (g >> 1) & 1u)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        *abort_flag = 1;
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
        }
    } else if (warp == 6) {
        // ------------------------------------------------------------ scale copier.
        // One thread issues every tcgen05 instruction it is given at ~60 cycles apiece; with the 12 scale
        // copies of a stage on the MMA thread that thread, not the weight stream, set the pace.  Here they
        // run one stage ahead into the other set of scale columns.  The copies do not depend on the tile, so
        // this lane only needs the number of stages its CTA walks.
        if (lane == 0) {
            int total = 0;
            {
                int ph = p_first;
                for (int u = unit_lo; u < unit_hi; ++u) {
                    const Unit un = decode_unit(P, u, ph);
                    total += un.ks1 - un.ks0;
                }
            }
            const uint32_t base16 = smem_u32(smem) >> 4;
            const uint32_t stage16 = static_cast<uint32_t>(kStageBytes) >> 4;
            const uint32_t off_sfb16 = static_cast<uint32_t>(kWBlock + NB * 128) >> 4;
            int s = 0;
            uint32_t full_phase = 0, lo0 = base16;
            for (int g = 0; g < total && !*abort_flag; ++g) {
                const uint32_t set = g & 1;
                if (!mbar_wait_bounded(&ctl->full[s], full_phase) ||
                    (g >= 2 && !mbar_wait_bounded(&ctl->sf_empty[set], ((g >> 1) - 1) & 1))) {
                    record_error(kErrGemmTmaBarrierTimeout);
                    *abort_flag = 1;
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
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
        const int q = warp & 3;
        const int et = q * 32 + lane;            // 0..127: the weight row inside the tile
        int unit_iter = 0, ph = p_first;
        pdl_wait_prior_grids();                   // the output buffer may still be read by the previous kernel
        for (int u = unit_lo; u < unit_hi && !*abort_flag; ++unit_iter) {
            const Group un = decode_group(P, u, unit_hi, ph);
            u = un.next;
            const TcProblem& pr = P.prob[un.p];
            const int buf = unit_iter & 1;
            if (!mbar_wait_bounded(&ctl->acc_full[buf], (unit_iter >> 1) & 1)) {
                record_error(kErrGemmMmaBarrierTimeout);
                *abort_flag = 1;
                break;
            }
            tc::fence_after_thread_sync();
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * 128;
            float v[2][16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int t = 0; t < 16; ++t) v[h][t] = 0.0f;
                for (int pc = 0; pc < P.pieces; ++pc) {
                    uint32_t r[16];
                    tmem_ld_32x32b_x16(taddr + h * kMaxNB + pc * 16, r);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int t = 0; t < 16; ++t) v[h][t] += __uint_as_float(r[t]);
                }
            }
            tc::fence_before_thread_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);

            const int n_pad = pr.row_tiles * 256;
            bool finalize = true;
            if (un.split0 != 0 || un.split1 != pr.splits - 1) {
                // this group covers only part of the tile's K range: hand its sums over.  The tile's groups
                // start at its first unit and wherever a CTA's range begins inside it.
                const int t0 = pr.unit_begin + un.rt * pr.splits;
                const long long total = P.total_units;
                const int grid = gridDim.x;
                const int b_first = static_cast<int>((static_cast<long long>(t0) * grid) / total) + 1;
                int ngroups = 1;
                for (int b = b_first; b < grid && static_cast<int>(b * total / grid) < t0 + pr.splits; ++b) {
                    if (static_cast<int>(b * total / grid) > t0) ++ngroups;
                }
                float* part = P.scratch + pr.scratch_off;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int n = un.rt * 256 + h * 128 + et;
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        if (t < P.M) part[(static_cast<size_t>(un.split0) * 16 + t) * n_pad + n] = v[h][t];
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (et == 0) ctl->ticket = atomicAdd(P.counters + pr.counter_off + un.rt, 1);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                finalize = (ctl->ticket == ngroups - 1);
                if (finalize) {
                    __threadfence();
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int n = un.rt * 256 + h * 128 + et;
#pragma unroll
                        for (int t = 0; t < 16; ++t) {
                            if (t < P.M) {
                                float acc = __ldcg(part + static_cast<size_t>(t) * n_pad + n);       // group at split 0
                                for (int b = b_first; b < grid && static_cast<int>(b * total / grid) < t0 + pr.splits; ++b) {
                                    const int sp = static_cast<int>(b * total / grid) - t0;
                                    if (sp > 0) acc += __ldcg(part + (static_cast<size_t>(sp) * 16 + t) * n_pad + n);
                                }
                                v[h][t] = acc;
                            }
                        }
                    }
                    if (et == 0) P.counters[pr.counter_off + un.rt] = 0;   // ready for the next launch
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");              // ticket slot free for the next unit
            }
            if (finalize) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int n = un.rt * 256 + h * 128 + et;
                    if (n >= pr.N) continue;
#pragma unroll
                    for (int t = 0; t < 16; ++t) {
                        if (t < P.M) {
                            float f = v[h][t] * pr.global_scale * __ldg(pr.row_scale + t);
                            if (pr.bias != nullptr) f += load_as_float(pr.bias, P.bias_dtype, n);
                            f = apply_activation(f, P.activation);
                            store_from_float(pr.out, P.out_dtype, static_cast<size_t>(t) * pr.ldo + n, f);
                        }
                    }
                }
            }
        }
    }

    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// Activation pieces in the tiled image: one CTA per token row t < 16 (rows >= M are zeroed).
// Same arithmetic as nvfp4_quantize_pieces_kernel in nvfp4_gemm.cu.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t e2m1_index(float a) {
    return (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) + (a > 3.5f) + (a > 5.0f);
}

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
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);
        e = 11 - ex;
    }
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
// Host side
// ---------------------------------------------------------------------------------------------
namespace {

struct TcPlan {
    int splits[TPB200_MAX_GROUP];
    int stages_per_split[TPB200_MAX_GROUP];
    size_t scratch_floats;
    size_t counters;
    int total_units;
};

// shared by the workspace query and the launch so that both see the same layout
int make_plan(const tpb200_gemv_tc_problem* probs, int count, int sms, TcPlan& plan) {
    long long total_stages = 0;
    for (int i = 0; i < count; ++i) {
        if (probs[i].N < 1 || probs[i].K < 16 || probs[i].K % 16 != 0) return TPB200_ERR_SHAPE;
        const long long row_tiles = (probs[i].N + 255) / 256;
        total_stages += row_tiles * ((probs[i].K + 255) / 256);
    }
    // aim for ~4 units per SM, units of 1..8 stages, and never longer than the shortest problem's K so
    // that the units of a mixed launch carry (nearly) the same number of stages: CTAs own equal COUNTS
    int target = static_cast<int>(std::min<long long>(8, std::max<long long>(1, total_stages / (4LL * sms))));
    for (int i = 0; i < count; ++i) target = std::min(target, (probs[i].K + 255) / 256);
    plan.scratch_floats = 0;
    plan.counters = 0;
    plan.total_units = 0;
    for (int i = 0; i < count; ++i) {
        const int row_tiles = (probs[i].N + 255) / 256;
        const int k_stages = (probs[i].K + 255) / 256;
        int splits = (k_stages + target - 1) / target;
        const int sps = (k_stages + splits - 1) / splits;
        splits = (k_stages + sps - 1) / sps;
        plan.splits[i] = splits;
        plan.stages_per_split[i] = sps;
        if (splits > 1) {
            plan.scratch_floats += static_cast<size_t>(splits) * 16 * row_tiles * 256;
            plan.counters += row_tiles;
        }
        plan.total_units += row_tiles * splits;
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

}  // namespace

extern "C" size_t tpb200_nvfp4_gemv_tc_workspace_size(const tpb200_gemv_tc_problem* problems, int count) {
    if (problems == nullptr || count < 1 || count > TPB200_MAX_GROUP) return 0;
    int sms = 0;
    if (device_sms(sms) != TPB200_OK) return 0;
    TcPlan plan;
    if (make_plan(problems, count, sms, plan) != TPB200_OK) return 0;
    // counters first (zero-initialised by the caller once), then the partial sums
    return (plan.counters * sizeof(int) + 255) / 256 * 256 + plan.scratch_floats * sizeof(float) + 256;
}

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
                                    size_t workspace_bytes, int flags, tpb200_stream_t stream) {
    TPB_REQUIRE(problems != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_GROUP, TPB200_ERR_SHAPE);
    TPB_REQUIRE(M >= 1 && M <= 16 && pieces >= 1 && pieces <= 4, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_valid_dtype(bias_dtype) && tpb_valid_dtype(out_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE(activation >= TPB200_ACT_NONE && activation <= TPB200_ACT_SILU, TPB200_ERR_ENUM);
    TPB_REQUIRE((flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    int sms = 0;
    if (device_sms(sms) != TPB200_OK) return TPB200_ERR_CUDA;
    TcPlan plan;
    const int st = make_plan(problems, count, sms, plan);
    if (st != TPB200_OK) return st;
    const size_t counter_bytes = (plan.counters * sizeof(int) + 255) / 256 * 256;
    if (plan.scratch_floats > 0) {
        TPB_REQUIRE(workspace != nullptr, TPB200_ERR_WORKSPACE);
        TPB_REQUIRE(workspace_bytes >= counter_bytes + plan.scratch_floats * sizeof(float), TPB200_ERR_WORKSPACE);
        TPB_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, TPB200_ERR_ALIGN);
    }

    tpb::TcParams P;
    P.num_problems = count;
    P.total_units = plan.total_units;
    P.M = M;
    P.pieces = pieces;
    P.bias_dtype = bias_dtype;
    P.out_dtype = out_dtype;
    P.activation = activation;
    P.counters = static_cast<int*>(workspace);
    P.scratch = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + counter_bytes);
    int units = 0, coff = 0;
    size_t soff = 0;
    for (int i = 0; i < count; ++i) {
        const tpb200_gemv_tc_problem& h = problems[i];
        TPB_REQUIRE(h.w_image && h.x_image && h.x_row_scale && h.out, TPB200_ERR_NULL);
        TPB_REQUIRE(tpb_aligned16(h.w_image) && tpb_aligned16(h.x_image), TPB200_ERR_ALIGN);
        TPB_REQUIRE(h.ldo == 0 || h.ldo >= h.N, TPB200_ERR_SHAPE);
        tpb::TcProblem& d = P.prob[i];
        d.w_image = static_cast<const uint8_t*>(h.w_image);
        d.x_image = static_cast<const uint8_t*>(h.x_image);
        d.row_scale = h.x_row_scale;
        d.bias = h.bias;
        d.out = h.out;
        d.N = h.N;
        d.K = h.K;
        d.ldo = h.ldo == 0 ? h.N : h.ldo;
        d.global_scale = h.global_scale;
        d.k_stages = (h.K + 255) / 256;
        d.row_tiles = (h.N + 255) / 256;
        d.splits = plan.splits[i];
        d.stages_per_split = plan.stages_per_split[i];
        d.unit_begin = units;
        d.scratch_off = static_cast<int>(soff);
        d.counter_off = coff;
        units += d.row_tiles * d.splits;
        if (d.splits > 1) {
            soff += static_cast<size_t>(d.splits) * 16 * d.row_tiles * 256;
            coff += d.row_tiles;
        }
    }

    const size_t smem = tpb::num_stages(pieces) * tpb::stage_bytes(pieces) + sizeof(tpb::SharedControl) + 1024;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(tpb::nvfp4_gemv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(std::min(plan.total_units, sms), 1, 1);
    cfg.blockDim = dim3(tpb::kThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, tpb::nvfp4_gemv_tc_kernel, P) != cudaSuccess) return TPB200_ERR_CUDA;
    return TPB200_OK;
}

// ---------------------------------------------------------------------------------------------
// The same GEMV for callers that are not able to allocate device memory.
//
// tpb200_nvfp4_gemv_tc needs a workspace for its split-K partial sums and tile counters.  Some
// callers have nowhere to get one from: a TensorRT plugin whose enqueue() was not granted a
// workspace, a robot-control loop that must not touch the allocator once it is running, host code
// that is handed raw pointers and no allocator of the framework that owns them.  For them the
// scratch lives in the library image itself, in the array below.  Every GPU that loads the library
// carries these 16 MiB until the process exits.
//
// Host code must not hand `g_static_scratch` to a kernel directly: in host code that name is only a
// stand-in for the symbol, not a device address.  The address is looked up once per device with
// cudaGetSymbolAddress while that device is current.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;
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
    TPB_REQUIRE(problems != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(count >= 1 && count <= TPB200_MAX_GROUP, TPB200_ERR_SHAPE);
    int sms = 0;
    if (device_sms(sms) != TPB200_OK) return TPB200_ERR_CUDA;
    TcPlan plan;
    const int st = make_plan(problems, count, sms, plan);
    if (st != TPB200_OK) return st;
    const size_t counter_bytes = (plan.counters * sizeof(int) + 255) / 256 * 256;
    const size_t need = counter_bytes + plan.scratch_floats * sizeof(float);
    // larger problems than the built-in scratch can hold are refused, never truncated
    TPB_REQUIRE(need <= kStaticScratchBytes, TPB200_ERR_WORKSPACE);
    void* scratch = nullptr;
    const int sa = static_scratch_address(&scratch);
    if (sa != TPB200_OK) return sa;
    // The array keeps whatever the previous call left.  Only the tile counters have to start at
    // zero; the partial sums are always written before they are read.
    if (counter_bytes > 0 &&
        cudaMemsetAsync(scratch, 0, counter_bytes, reinterpret_cast<cudaStream_t>(stream)) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    return tpb200_nvfp4_gemv_tc(problems, count, M, pieces, bias_dtype, out_dtype, activation, scratch,
                                kStaticScratchBytes, flags, stream);
}
