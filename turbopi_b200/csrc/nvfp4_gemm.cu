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
// No multicast, no cluster; every wait is bounded and reports through the device error word.
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "tcgen05.cuh"

namespace tpb {
namespace {

constexpr int kBM = 128;
constexpr int kBN = 128;
constexpr int kBKBytes = 128;            // 256 e2m1 codes per row per stage
constexpr int kMaxStages = 5;
constexpr int kMaxPieces = 4;
constexpr int kTile = 128 * kBKBytes;    // 16 KB operand tile
constexpr int kSfSlab = 4 * 512;         // 4 K-atoms of one 128-row tile
constexpr int kOutBuf = 128 * 128;       // one staged output box: 128 rows x 128 bytes
constexpr int kThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kAccCols = kBN;            // fp32 accumulator columns per buffer
constexpr uint32_t kSfbCol = 2 * kAccCols;
constexpr uint32_t kSfaCol = kSfbCol + 16;   // 16 columns per piece
constexpr int kSmemBudget = 227 * 1024 - 2048;

__host__ __device__ constexpr int stage_bytes(int pieces) { return (1 + pieces) * (kTile + kSfSlab); }
__host__ __device__ constexpr int num_stages(int pieces) {
    return (kSmemBudget - 2 * kOutBuf) / stage_bytes(pieces) < kMaxStages
               ? (kSmemBudget - 2 * kOutBuf) / stage_bytes(pieces)
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
    int debug;   // development switches (TPB200_GEMM_DEBUG): 1 = no stores, 2 = no accumulator reads, 4 = no MMA
};

enum { kEpiPlain = 0, kEpiQkvRope = 1 };

struct SharedControl {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

// epilogue activations with the hardware approximations (results are rounded to bf16 anyway)
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(inner));
    return 0.5f * x * (1.0f + t);
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

// 16-byte chunk c of row r in a staged 128-byte-row box (the layout a 128B-swizzled TMA store reads)
__device__ __forceinline__ uint8_t* staged_chunk(uint8_t* buf, int r, int c) {
    return buf + r * 128 + ((c ^ (r & 7)) << 4);
}

__global__ void __launch_bounds__(kThreads, 1) nvfp4_gemm_kernel(const __grid_constant__ GemmParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int pieces = P.a_pieces;
    const int nstages = num_stages(pieces);
    const int stage_sz = stage_bytes(pieces);
    // stage layout: [B tile][A tile x pieces][SFB slab][SFA slab x pieces]
    const int off_a = kTile;
    const int off_sfb = (1 + pieces) * kTile;
    const int off_sfa = off_sfb + kSfSlab;
    uint8_t* out_stage = smem + nstages * stage_sz;                       // 2 x 16 KB, 1024-byte aligned
    SharedControl* ctl = reinterpret_cast<SharedControl*>(out_stage + 2 * kOutBuf);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = P.m_blocks * P.n_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&ctl->full[s], 1);
            mbar_init(&ctl->empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&ctl->acc_full[b], 1);
            mbar_init(&ctl->acc_empty[b], 4);
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

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tc::prefetch_tensormap(&P.map_a);
            tc::prefetch_tensormap(&P.map_b);
            const int sf_row_stride = P.k_stages * kSfSlab;   // bytes per 128-row tile of scales
            int it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                const int m_blk = tile % P.m_blocks;
                const int n_blk = tile / P.m_blocks;
                for (int ks = 0; ks < P.k_stages; ++ks, ++it) {
                    const int s = it % nstages;
                    if (it >= nstages && !mbar_wait_bounded(&ctl->empty[s], ((it / nstages) - 1) & 1)) {
                        record_error(kErrGemmEmptyBarrierTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    uint8_t* st = smem + s * stage_sz;
                    mbar_expect_tx(&ctl->full[s], stage_sz);
                    tc::tma_load_2d(st, &P.map_b, ks * kBKBytes, n_blk * kBN, &ctl->full[s]);
                    bulk_copy_g2s(st + off_sfb,
                                  P.sfb + static_cast<size_t>(n_blk) * sf_row_stride + static_cast<size_t>(ks) * kSfSlab,
                                  kSfSlab, &ctl->full[s]);
                    for (int p = 0; p < pieces; ++p) {
                        const int a_row_tile = p * (P.a_piece_rows >> 7) + m_blk;
                        tc::tma_load_2d(st + off_a + p * kTile, &P.map_a, ks * kBKBytes, a_row_tile * kBM, &ctl->full[s]);
                        bulk_copy_g2s(st + off_sfa + p * kSfSlab,
                                      P.sfa + static_cast<size_t>(a_row_tile) * sf_row_stride +
                                          static_cast<size_t>(ks) * kSfSlab,
                                      kSfSlab, &ctl->full[s]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = tc::make_idesc_mxf4nvf4(kBN);
            int it = 0, tile_iter = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tile_iter) {
                const int buf = tile_iter & 1;
                if (tile_iter >= 2 && !mbar_wait_bounded(&ctl->acc_empty[buf], ((tile_iter >> 1) - 1) & 1)) {
                    record_error(kErrGemmEpilogueBarrierTimeout);
                    *abort_flag = 1;
                    break;
                }
                tc::fence_after_thread_sync();
                const uint32_t tmem_acc = tmem_base + buf * kAccCols;
                for (int ks = 0; ks < P.k_stages; ++ks, ++it) {
                    const int s = it % nstages;
                    if (!mbar_wait_bounded(&ctl->full[s], (it / nstages) & 1)) {
                        record_error(kErrGemmTmaBarrierTimeout);
                        *abort_flag = 1;
                        break;
                    }
                    tc::fence_after_thread_sync();
                    const uint32_t st = smem_u32(smem + s * stage_sz);
#pragma unroll
                    for (int a = 0; a < 4; ++a) {
                        tc::cp_sf_32x128b(tmem_base + kSfbCol + 4 * a, tc::make_sf_desc(st + off_sfb + a * 512));
                    }
                    for (int p = 0; p < pieces; ++p) {
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            tc::cp_sf_32x128b(tmem_base + kSfaCol + 16 * p + 4 * a,
                                              tc::make_sf_desc(st + off_sfa + p * kSfSlab + a * 512));
                        }
#pragma unroll
                        for (int a = 0; a < 4; ++a) {
                            if (P.debug & 4) break;
                            tc::mma_mxf4nvf4(tmem_acc, tc::make_kmajor_sw128_desc(st + off_a + p * kTile, a * 32),
                                             tc::make_kmajor_sw128_desc(st, a * 32), idesc,
                                             tmem_base + kSfaCol + 16 * p + 4 * a, tmem_base + kSfbCol + 4 * a,
                                             (ks | p | a) != 0);
                        }
                    }
                    tc::commit(&ctl->empty[s]);   // stage s may be refilled once these MMAs have read it
                }
                tc::commit(&ctl->acc_full[buf]);  // accumulator complete
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..5, 128 threads)
        const int q = warp & 3;                       // tensor-memory lane quarter this warp may read
        const int row = q * 32 + lane;                // row of the tile this thread owns
        const bool issuer = (threadIdx.x == 64);      // first epilogue thread issues the TMA stores
        int tile_iter = 0;
        uint32_t nstore = 0;                          // staged boxes so far (buffer = nstore & 1)
        for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, ++tile_iter) {
            const int m_blk = tile % P.m_blocks;
            const int n_blk = tile / P.m_blocks;
            const int buf = tile_iter & 1;
            if (!mbar_wait_bounded(&ctl->acc_full[buf], (tile_iter >> 1) & 1)) {
                record_error(kErrGemmMmaBarrierTimeout);
                *abort_flag = 1;
                break;
            }
            tc::fence_after_thread_sync();
            const int m = m_blk * kBM + row;
            const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kAccCols;
            const float rs = (P.row_scale != nullptr && m < P.M) ? P.alpha * __ldg(P.row_scale + m) : P.alpha;
            if (P.debug & 2) {
                tc::fence_before_thread_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                continue;
            }
            if (P.epilogue == kEpiPlain) {
                // boxes of 128 bytes per row: 64 bf16 or 32 fp32 columns
                const int cols_per_box = P.out_dtype == TPB200_BF16 ? 64 : 32;
                const int nboxes = kBN / cols_per_box;
#pragma unroll 1
                for (int bx = 0; bx < nboxes; ++bx, ++nstore) {
                    uint8_t* ob = out_stage + (nstore & 1) * kOutBuf;
                    if (issuer) bulk_wait_group_read<1>();    // the store that last used this buffer has read it
                    epilogue_barrier();
                    const int n0 = n_blk * kBN + bx * cols_per_box;
#pragma unroll 1
                    for (int c = 0; c < cols_per_box / 32; ++c) {
                        uint32_t r[32];
                        if (!(P.debug & 16)) {
                            tc::tmem_ld_32x32b_x32(taddr + bx * cols_per_box + c * 32, r);
                            tc::tmem_ld_wait();
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = i + row;
                        }
                        if (P.debug & 8) {
                            if (r[5] == 0x7fc12345u) record_error(999);
                            continue;
                        }
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]) * rs;
                        if (P.bias != nullptr) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                if (n0 + c * 32 + i < P.N) v[i] += __ldg(P.bias + n0 + c * 32 + i);
                            }
                        }
                        // one uniform branch per chunk: the transcendental code stays out of the plain path
                        if (P.activation == TPB200_ACT_GELU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_fast(v[i]);
                        } else if (P.activation == TPB200_ACT_SILU) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = silu_fast(v[i]);
                        }
                        if (P.out_dtype == TPB200_BF16) {
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                uint32_t w[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(v[g * 8 + 2 * i], v[g * 8 + 2 * i + 1]);
                                    w[i] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                *reinterpret_cast<uint4*>(staged_chunk(ob, row, c * 4 + g)) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                *reinterpret_cast<float4*>(staged_chunk(ob, row, g)) =
                                    make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                            }
                        }
                    }
                    if (bx == nboxes - 1) {
                        // everything this warp needs from the accumulator is in registers / shared memory
                        tc::fence_before_thread_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                    }
                    fence_proxy_async_smem();
                    epilogue_barrier();
                    if (issuer) {
                        if (!(P.debug & 1)) tma_store_2d(&P.map_out, ob, n0, m_blk * kBM);
                        bulk_commit_group();
                    }
                }
            } else {
                // Fused QKV: tile columns [0,64) are head offsets i0..i0+63, columns [64,128) their
                // rotation partners i + 128.  bf16 arithmetic as torch does it: q, cos, sin in bf16,
                // each product and the sum rounded to bf16.  Two boxes of 64 columns: lo and hi.
                const int head = n_blk >> 1;
                const int i0 = (n_blk & 1) * 64;
                const int n_heads_q = P.q_dim >> 8;
                const bool is_v = head == n_heads_q + 1;
                const int pos = (m < P.M) ? __ldg(P.positions + m) : 0;
                uint8_t* ob_lo = out_stage;
                uint8_t* ob_hi = out_stage + kOutBuf;
                if (issuer) bulk_wait_group_read<0>();
                epilogue_barrier();
#pragma unroll 1
                for (int c = 0; c < 2; ++c) {
                    uint32_t lo[32], hi[32];
                    tc::tmem_ld_32x32b_x32(taddr + c * 32, lo);
                    tc::tmem_ld_32x32b_x32(taddr + 64 + c * 32, hi);
                    tc::tmem_ld_wait();
                    if (c == 1) {
                        tc::fence_before_thread_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&ctl->acc_empty[buf]);
                    }
                    const int i = i0 + c * 32;   // head offset of lo[0]
                    const uint4* cs = reinterpret_cast<const uint4*>(P.rope_cos + static_cast<size_t>(pos) * 128 + i);
                    const uint4* sn = reinterpret_cast<const uint4*>(P.rope_sin + static_cast<size_t>(pos) * 128 + i);
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 cv = make_uint4(0, 0, 0, 0), sv = make_uint4(0, 0, 0, 0);
                        if (!is_v) { cv = __ldg(cs + g); sv = __ldg(sn + g); }
                        const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w};
                        const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
                        uint32_t olo[4], ohi[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int e = g * 8 + 2 * j;
                            __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(lo[e]) * rs, __uint_as_float(lo[e + 1]) * rs);
                            __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(hi[e]) * rs, __uint_as_float(hi[e + 1]) * rs);
                            if (!is_v) {
                                const __nv_bfloat162 co = *reinterpret_cast<const __nv_bfloat162*>(&cw[j]);
                                const __nv_bfloat162 si = *reinterpret_cast<const __nv_bfloat162*>(&sw[j]);
                                // first half: x*cos + (-x_partner)*sin ; second half: x_partner*cos + x*sin
                                const __nv_bfloat162 ra = __hadd2(__hmul2(a, co), __hmul2(__hneg2(b), si));
                                const __nv_bfloat162 rb = __hadd2(__hmul2(b, co), __hmul2(a, si));
                                a = ra;
                                b = rb;
                            }
                            olo[j] = *reinterpret_cast<uint32_t*>(&a);
                            ohi[j] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        *reinterpret_cast<uint4*>(staged_chunk(ob_lo, row, c * 4 + g)) = make_uint4(olo[0], olo[1], olo[2], olo[3]);
                        *reinterpret_cast<uint4*>(staged_chunk(ob_hi, row, c * 4 + g)) = make_uint4(ohi[0], ohi[1], ohi[2], ohi[3]);
                    }
                }
                fence_proxy_async_smem();
                epilogue_barrier();
                if (issuer) {
                    if (!(P.debug & 1)) {
                        const CUtensorMap* map = head < n_heads_q ? &P.map_out : (is_v ? &P.map_v : &P.map_k);
                        const int x0 = head < n_heads_q ? head * 256 + i0 : i0;
                        tma_store_2d(map, ob_lo, x0, m_blk * kBM);
                        tma_store_2d(map, ob_hi, x0 + 128, m_blk * kBM);
                    }
                    bulk_commit_group();
                }
                nstore += 2;
            }
        }
        if (issuer) bulk_wait_group_all();   // every output tile has landed before the CTA goes away
    }

    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem_base, kTmemCols);
    }
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

extern "C" int tpb200_nvfp4_gemm_ex(const tpb200_nvfp4_gemm_args* a, tpb200_stream_t stream) {
    TPB_REQUIRE(a != nullptr, TPB200_ERR_NULL);
    const int M = a->M, N = a->N, K = a->K;
    TPB_REQUIRE(a->a_packed && a->a_sf && a->b_packed && a->b_sf, TPB200_ERR_NULL);
    TPB_REQUIRE(M >= 1 && N >= 8 && N % 8 == 0 && K >= 16 && K % 16 == 0, TPB200_ERR_SHAPE);
    TPB_REQUIRE(a->activation >= TPB200_ACT_NONE && a->activation <= TPB200_ACT_SILU, TPB200_ERR_ENUM);
    TPB_REQUIRE(a->a_pitch >= K / 2 && a->b_pitch >= K / 2 && a->a_pitch % 16 == 0 && a->b_pitch % 16 == 0,
                TPB200_ERR_ALIGN);
    TPB_REQUIRE(tpb_aligned16(a->a_packed) && tpb_aligned16(a->b_packed) && tpb_aligned16(a->a_sf) &&
                    tpb_aligned16(a->b_sf),
                TPB200_ERR_ALIGN);
    const int pieces = a->a_pieces <= 0 ? 1 : a->a_pieces;
    TPB_REQUIRE(pieces <= 4, TPB200_ERR_SHAPE);
    TPB_REQUIRE(pieces == 1 || (a->a_piece_rows >= M && a->a_piece_rows % 128 == 0), TPB200_ERR_SHAPE);
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
        TPB_REQUIRE(a->ldo >= N, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(a->out) && (static_cast<long long>(a->ldo) * tpb_dtype_size(a->out_dtype)) % 16 == 0,
                    TPB200_ERR_ALIGN);
    }

    tpb::GemmParams P;
    const uint64_t a_rows = pieces == 1 ? static_cast<uint64_t>(M) : static_cast<uint64_t>(pieces) * a->a_piece_rows;
    if (!tpb::make_tensor_map_bytes_sw128(&P.map_a, a->a_packed, static_cast<uint64_t>(K) / 2, a_rows, a->a_pitch,
                                          tpb::kBM) ||
        !tpb::make_tensor_map_bytes_sw128(&P.map_b, a->b_packed, static_cast<uint64_t>(K) / 2, N, a->b_pitch,
                                          tpb::kBN)) {
        return TPB200_ERR_CUDA;
    }
    if (qkv) {
        if (!tpb::make_tensor_map_out_sw128(&P.map_out, a->qkv_q_out, TPB200_BF16, a->qkv_q_dim, M,
                                            static_cast<uint64_t>(a->qkv_ldq) * 2) ||
            !tpb::make_tensor_map_out_sw128(&P.map_k, a->qkv_k_rows, TPB200_BF16, 256, M, 512) ||
            !tpb::make_tensor_map_out_sw128(&P.map_v, a->qkv_v_rows, TPB200_BF16, 256, M, 512)) {
            return TPB200_ERR_CUDA;
        }
    } else {
        if (!tpb::make_tensor_map_out_sw128(&P.map_out, a->out, a->out_dtype, N, M,
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
    P.n_blocks = (N + tpb::kBN - 1) / tpb::kBN;
    P.a_pieces = pieces;
    P.a_piece_rows = pieces == 1 ? 0 : a->a_piece_rows;
    P.row_scale = a->a_row_scale;
    P.epilogue = qkv ? tpb::kEpiQkvRope : tpb::kEpiPlain;
    P.q_dim = a->qkv_q_dim;
    P.positions = a->qkv_positions;
    P.rope_cos = static_cast<const __nv_bfloat16*>(a->qkv_rope_cos);
    P.rope_sin = static_cast<const __nv_bfloat16*>(a->qkv_rope_sin);
    {
        const char* dbg = getenv("TPB200_GEMM_DEBUG");
        P.debug = dbg != nullptr ? atoi(dbg) : 0;
    }

    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    const size_t smem = tpb::num_stages(pieces) * tpb::stage_bytes(pieces) + 2 * tpb::kOutBuf + sizeof(tpb::SharedControl) + 1024;
    static std::atomic<uint64_t> configured{0};
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(tpb::nvfp4_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 227 * 1024) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    const int grid = std::min(P.m_blocks * P.n_blocks, sms);
    tpb::nvfp4_gemm_kernel<<<grid, tpb::kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(P);
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
