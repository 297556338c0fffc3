// Attention for the Pi0.5 shapes on the tensor cores (tcgen05 kind::f16, bf16 operands, fp32 accumulators
// in tensor memory):
//
//   Gemma prefix / action expert   8 query heads on ONE key/value head, head_dim 256: the (token, head)
//                                  pairs are just rows of a [tokens * 8, 256] matrix that all attend to the
//                                  same keys, so the call is single-head attention over that matrix
//                                  (712 x 8 rows on 712 keys; 50 x 8 rows on 762 keys), with an additive
//                                  bias per key for padded prompt tokens / a missing camera;
//   SigLIP                         2 images x 16 heads, 256 tokens, head_dim 72 (padded to 128 in shared memory).
//
// Every problem is far too small to fill the machine with one CTA per 128 query rows running over all
// keys (the action expert has 4 such tiles), so the keys are split too: CTA (row tile, key tile of 256,
// group) computes S = Q K^T as two 128-key tiles side by side in tensor memory (2 x 16 MMAs of K = 16), the
// softmax of its 128 x 256 block relative to the block's own row maxima (base-2 exponentials, 256 threads:
// two per row), and O = P V (16 MMAs), and leaves O, the row maxima and the row sums in scratch; a second
// small kernel combines the key tiles' partial results (the usual log-sum-exp merge).  With a single key
// tile the first kernel writes the final rows itself.
//
// Operands in shared memory, all in the 128-byte-swizzle image (rows of 128 B = 64 bf16, 16-byte chunk c of
// row r at c ^ (r & 7), 8-row groups 1024 B apart, one 16 KB block per 64 columns of head_dim):
//   Q [128 rows][D], K [2 x 128 keys][D]  K-major operands of S = Q K^T
//   P [128 rows][256 keys]                K-major A operand of O = P V, written by the softmax threads over Q
//   V [2 x 128 keys][D]                   loaded where K was once the S MMAs are done; the SAME image is read as an
//                                         MN-major B operand (the 128-byte direction is head_dim = N, the rows
//                                         are keys = K): no transposed copy of V.
// Loads are TMA tile copies through 4-dimensional tensor maps (head_dim, rows, groups; zero fill past the end
// of a matrix), issued by one thread; the partial O of a CTA is staged where V was and leaves as one bulk
// copy.  Nothing here waits on another CTA; every wait is bounded and reports through the device error word.
#include <algorithm>
#include <atomic>

#include "tcgen05.cuh"

namespace tpb {
namespace {

constexpr int kRows = 128;              // query rows per CTA
constexpr int kKeyTile = 128;           // keys per S tile (one MMA's N)
constexpr int kKeysCta = 256;           // keys per CTA: two S tiles side by side in tensor memory
constexpr int kChunkBytes = kRows * 128;   // one 64-column block of an operand
constexpr int kThreadsAttn = 256;           // two warps per 32-lane quarter of tensor memory: each takes half the columns
constexpr float kMasked = -2.3819763e38f;   // the reference's additive mask value (pi0_pytorch.py:185-188)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kFloor2 = -3.0e38f;         // lowest score in the base-2 domain (the mask value times log2 e overflows)
constexpr uint32_t kTmemColsAttn = 512;
constexpr uint32_t kColS = 0, kColO = 256;
constexpr long long kWaitCycles = 200000000LL;   // ~0.1 s: bound of each wait for copies / tensor cores

// One operand (q, k or v) as a 4-dimensional tensor map: dimension 0 is head_dim, the other three are the
// rows and the two group indices ordered by ascending stride; slot[i] is the coordinate position (1..3)
// of rows / inner group / outer group, mul[i] is 0 for a broadcast (stride 0) group dimension.
struct AttnOperand {
    CUtensorMap map;
    int slot[3];
    int mul[3];
};

struct AttnParams {
    AttnOperand q, k, v;
    __nv_bfloat16* out;
    const __nv_bfloat16* key_bias;
    int n_rows, n_keys, head_dim, dpad;         // dpad: head_dim rounded up to 64
    int ldo;
    int groups_inner;
    long long o_stride[2];
    float scale2;                               // scale * log2(e): the softmax runs in base 2
    int row_tiles, key_tiles;
    int keys_per_cta;                           // 256 (two S tiles), or 128 when the problem has few CTAs
    float* part_o;                              // [group][row tile][key tile] images of 128 rows x dvp floats
    float* part_ml;                             // [group][row tile][key tile][128][2]
    int dv;                                     // head_dim rounded up to 16: N of the second MMA
    int dvp;                                    // head_dim rounded up to 32: row pitch of a partial image
    // optional: the merged rows also leave as the tiled A image of the tensor-core GEMM that follows
    // (token = rows_per_token consecutive rows = one row of the image, K = rows_per_token * head_dim)
    uint8_t* qa_image;
    float* qa_row_scale;
    int qa_pieces;
    int qa_rows_per_token;
    uint8_t* qa_sf;          // not null: the row-major operand form (codes [pieces * piece_rows, pitch] + scale atoms)
    int qa_pitch, qa_piece_rows;
};

struct AttnControl {
    uint64_t bar_k0, bar_k1, bar_s, bar_v, bar_o;
    uint32_t tmem_base;
    float bias2[kKeysCta];
    float half_max[2][kRows];                   // row maxima / row sums of the two column halves
    float half_sum[2][kRows];
};

// Instruction descriptor for kind::f16 with bf16 operands and an fp32 accumulator, M = 128:
//   [4,6) D format = 1 (f32)  [7,10) A format = 1 (bf16)  [10,13) B format = 1  [15] A major  [16] B major
//   (0 = K-major, 1 = MN-major)  [17,23) N >> 3  [24,29) M >> 4
__host__ __device__ constexpr uint32_t make_idesc_bf16(int n, int b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(b_mn_major) << 16) |
           (static_cast<uint32_t>(n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 128 rows starting at `row0` of group (ga, gb): one 64-column box per 16 KB block of the swizzled image
__device__ __forceinline__ void load_rows(uint8_t* dst, const AttnOperand& op, int row0, int ga, int gb, int nchunk,
                                          uint64_t* bar) {
    const int v[3] = {row0 * op.mul[0], gb * op.mul[1], ga * op.mul[2]};
    int c1 = 0, c2 = 0, c3 = 0;
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        c1 = op.slot[i] == 1 ? v[i] : c1;
        c2 = op.slot[i] == 2 ? v[i] : c2;
        c3 = op.slot[i] == 3 ? v[i] : c3;
    }
    for (int c = 0; c < nchunk; ++c) tc::tma_load_4d(dst + c * kChunkBytes, &op.map, c * 64, c1, c2, c3, bar);
}

__device__ __forceinline__ void bulk_store_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kThreadsAttn, 1) attention_partial_kernel(const __grid_constant__ AttnParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int nchunk = P.dpad >> 6;
    uint8_t* sQ = smem;                                   // later P: 128 rows x 256 keys = four 64-key blocks
    uint8_t* sKV = sQ + max(nchunk, 4) * kChunkBytes;     // two key tiles: K first, then V, then the staged partial O
    const uint32_t tile_bytes = static_cast<uint32_t>(nchunk) * kChunkBytes;
    AttnControl* ctl = reinterpret_cast<AttnControl*>(sKV + 2 * tile_bytes);

    const int rt = blockIdx.x, kt = blockIdx.y, g = blockIdx.z;
    const int ga = g / P.groups_inner, gb = g - ga * P.groups_inner;
    const int warp = threadIdx.x >> 5;
    const int key0 = kt * P.keys_per_cta;
    const int nt = (P.keys_per_cta > kKeyTile && P.n_keys - key0 > kKeyTile) ? 2 : 1;  // S tiles of this CTA

    if (threadIdx.x == 0) {
        mbar_init(&ctl->bar_k0, 1);
        mbar_init(&ctl->bar_k1, 1);
        mbar_init(&ctl->bar_s, 1);
        mbar_init(&ctl->bar_v, 1);
        mbar_init(&ctl->bar_o, 1);
        fence_mbar_init();
        tc::prefetch_tensormap(&P.q.map);
        tc::prefetch_tensormap(&P.k.map);
        tc::prefetch_tensormap(&P.v.map);
    }
    if (warp == 1) {
        // a whole, converged warp (not the one whose lane 0 just ran the barrier set-up on its own)
        __syncwarp();
        tc::tmem_alloc(&ctl->tmem_base, kTmemColsAttn);
        tc::tmem_relinquish();
    }
    pdl_launch_dependents();
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem = ctl->tmem_base;
    pdl_wait_prior_grids();                               // q, k, v (and the bias) may come from the previous kernel

    // warps 1..7: the keys' additive bias in the base-2 domain (visible to all after the barrier behind the S wait)
    for (int i = threadIdx.x - 32; i >= 0 && i < kKeysCta; i += kThreadsAttn - 32) {
        const int key = key0 + i;
        float b = kFloor2;                                // keys past the end never count
        if (key < P.n_keys) {
            b = P.key_bias != nullptr ? fmaxf(__bfloat162float(P.key_bias[key]) * kLog2e, kFloor2) : 0.0f;
        }
        ctl->bias2[i] = b;
    }

    // ---------------------------------------------------------------- loads, S = Q K^T (two key tiles)
    if (threadIdx.x == 0) {
        mbar_expect_tx(&ctl->bar_k0, 2 * tile_bytes);
        load_rows(sQ, P.q, rt * kRows, ga, gb, nchunk, &ctl->bar_k0);
        load_rows(sKV, P.k, key0, ga, gb, nchunk, &ctl->bar_k0);
        if (nt == 2) {
            mbar_expect_tx(&ctl->bar_k1, tile_bytes);
            load_rows(sKV + tile_bytes, P.k, key0 + kKeyTile, ga, gb, nchunk, &ctl->bar_k1);
        }
        const uint32_t idesc = make_idesc_bf16(kKeyTile, 0);
        const uint32_t q16 = smem_u32(sQ) >> 4;
        const int ksteps = (P.head_dim + 15) >> 4;        // 16 columns of head_dim per MMA
        bool loaded = true;
        for (int t = 0; t < nt && loaded; ++t) {
            loaded = mbar_wait_bounded(t == 0 ? &ctl->bar_k0 : &ctl->bar_k1, 0, kWaitCycles);
            if (!loaded) {
                record_error(kErrAttnBarrierTimeout);
                break;
            }
            tc::fence_after_thread_sync();
            const uint32_t k16 = (smem_u32(sKV) + t * tile_bytes) >> 4;
            for (int kk = 0; kk < ksteps; ++kk) {
                const uint32_t off = static_cast<uint32_t>((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4;
                mma_bf16(tmem + kColS + t * kKeyTile, tc::desc_from_words(q16 + off, tc::kDescHiKmajorSw128),
                         tc::desc_from_words(k16 + off, tc::kDescHiKmajorSw128), idesc, kk > 0 ? 1u : 0u);
            }
        }
        if (loaded) tc::commit(&ctl->bar_s);              // otherwise the wait below runs out for the whole CTA
    }
    // every wait is short (the work behind it takes microseconds) and its outcome is made uniform over the CTA:
    // the tensor-memory loads below are warp-collective
    bool ok = mbar_wait_bounded(&ctl->bar_s, 0, 2 * kWaitCycles);
    if (!ok) record_error(kErrAttnBarrierTimeout);
    ok = __syncthreads_and(ok);
    tc::fence_after_thread_sync();

    // the S MMAs have read K: V takes its place while the softmax runs
    if (threadIdx.x == 0 && ok) {
        mbar_expect_tx(&ctl->bar_v, nt * tile_bytes);
        load_rows(sKV, P.v, key0, ga, gb, nchunk, &ctl->bar_v);
        if (nt == 2) load_rows(sKV + tile_bytes, P.v, key0 + kKeyTile, ga, gb, nchunk, &ctl->bar_v);
    }

    // ---------------------------------------------------------------- softmax of this block, P -> shared memory
    // Thread (half, row): the row's scores in columns [64 * half, 64 * half + 64) of each S tile.
    const int row = threadIdx.x & (kRows - 1);            // tensor-memory lane = query row of the tile
    const int half = threadIdx.x >> 7;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    float m = kFloor2;
    float l = 0.0f;
    if (ok) {
        // pass 1: the maximum over this thread's up to 128 scores (base-2 domain), all loads in flight at once
        for (int t = 0; t < nt; ++t) {
            uint32_t r[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tc::tmem_ld_32x32b_x32(lane_addr + kColS + t * kKeyTile + half * 64 + c * 32, r[c]);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    m = fmaxf(m, fmaf(__uint_as_float(r[c][j]), P.scale2, ctl->bias2[t * kKeyTile + half * 64 + c * 32 + j]));
                }
            }
        }
        ctl->half_max[half][row] = m;
    }
    __syncthreads();
    if (ok) {
        m = fmaxf(m, ctl->half_max[half ^ 1][row]);
        // pass 2: p = 2^(t - m) rounded to bf16 (what the PyTorch path feeds its second matmul), row sum of the
        // rounded values, 16-byte stores into the K-major image of P
        uint8_t* sP = sQ;
        for (int t = 0; t < nt; ++t) {
            uint32_t r[2][32];
#pragma unroll
            for (int c = 0; c < 2; ++c) tc::tmem_ld_32x32b_x32(lane_addr + kColS + t * kKeyTile + half * 64 + c * 32, r[c]);
            tc::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
#pragma unroll
                for (int j8 = 0; j8 < 4; ++j8) {
                    uint32_t w[4];
#pragma unroll
                    for (int j2 = 0; j2 < 4; ++j2) {
                        const int j = j8 * 8 + j2 * 2;
                        const float* b2 = &ctl->bias2[t * kKeyTile + half * 64 + c * 32 + j];
                        const float x0 = fmaf(__uint_as_float(r[c][j]), P.scale2, b2[0]) - m;
                        const float x1 = fmaf(__uint_as_float(r[c][j + 1]), P.scale2, b2[1]) - m;
                        const __nv_bfloat162 pb = __floats2bfloat162_rn(ex2(x0), ex2(x1));
                        l += __bfloat162float(pb.x) + __bfloat162float(pb.y);
                        w[j2] = *reinterpret_cast<const uint32_t*>(&pb);
                    }
                    const int ch = t * 16 + half * 8 + c * 4 + j8;   // 16-byte chunk of the 256-key row: 0..31
                    uint8_t* dst = sP + (ch >> 3) * kChunkBytes + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
        }
        ctl->half_sum[half][row] = l;
    }
    fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    if (ok) l += ctl->half_sum[half ^ 1][row];

    // ---------------------------------------------------------------- O = P V
    if (threadIdx.x == 0 && ok) {
        if (mbar_wait_bounded(&ctl->bar_v, 0, kWaitCycles)) {
            tc::fence_after_thread_sync();
            const uint32_t idesc = make_idesc_bf16(P.dv, 1);  // B = V read MN-major
            const uint32_t p16 = smem_u32(sQ) >> 4;
            // MN-major, 128-byte swizzle: 64 columns of head_dim are contiguous, 8-key groups 1024 B apart
            // (stride offset), the next 64 columns one 16 KB block further (leading offset)
            constexpr uint32_t kDescHiMnSw128 = (1024u >> 4) | (1u << 14) | (static_cast<uint32_t>(tc::kSwizzle128B) << 29);
            constexpr uint32_t kLboField = (static_cast<uint32_t>(kChunkBytes) >> 4) << 16;
            for (int kk = 0; kk < nt * (kKeyTile / 16); ++kk) {
                const uint32_t a_off = static_cast<uint32_t>((kk >> 2) * kChunkBytes + (kk & 3) * 32) >> 4;
                const uint32_t v16 = (smem_u32(sKV) + (kk >> 3) * tile_bytes + (kk & 7) * 2048) >> 4;
                mma_bf16(tmem + kColO, tc::desc_from_words(p16 + a_off, tc::kDescHiKmajorSw128),
                         tc::desc_from_words(v16 | kLboField, kDescHiMnSw128), idesc, kk > 0 ? 1u : 0u);
            }
            tc::commit(&ctl->bar_o);
        } else {
            record_error(kErrAttnBarrierTimeout);         // the wait below runs out for the whole CTA
        }
    }
    if (ok) {
        ok = mbar_wait_bounded(&ctl->bar_o, 0, 2 * kWaitCycles);
        if (!ok) record_error(kErrAttnBarrierTimeout);
    }
    ok = __syncthreads_and(ok);
    tc::fence_after_thread_sync();

    // ---------------------------------------------------------------- write the rows
    // The tensor-memory loads are warp-collective: every lane executes them, rows past the end of the matrix
    // only skip the stores.  With a single key tile the rows are final (bf16, normalised); otherwise the
    // unnormalised fp32 rows are staged in shared memory where V was (chunk c of row r at c ^ (r & 7), so the
    // stores of a quarter warp spread over all banks) and leave as ONE bulk copy, image and all.
    const int grow = rt * kRows + row;
    const bool store = grow < P.n_rows;
    const bool final_rows = P.key_tiles == 1 && P.qa_image == nullptr;
    const size_t tile = (static_cast<size_t>(g) * P.row_tiles + rt) * P.key_tiles + kt;
    if (ok) {
        __nv_bfloat16* o = P.out + ga * P.o_stride[0] + gb * P.o_stride[1] + static_cast<size_t>(store ? grow : 0) * P.ldo;
        uint8_t* srow = sKV + static_cast<size_t>(row) * P.dvp * 4;
        if (!final_rows && store && half == 0) {
            float* pml = P.part_ml + (tile * kRows + row) * 2;
            pml[0] = m;
            pml[1] = l;
        }
        const float inv = 1.0f / l;
        for (int c64 = half * 64; c64 < P.dv; c64 += 128) {   // the halves take alternate 64-column batches
            // up to four 16-column loads in flight, one wait
            uint32_t r4[4][16];
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                if (c64 + q4 * 16 < P.dv) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                        : "=r"(r4[q4][0]), "=r"(r4[q4][1]), "=r"(r4[q4][2]), "=r"(r4[q4][3]), "=r"(r4[q4][4]), "=r"(r4[q4][5]),
                          "=r"(r4[q4][6]), "=r"(r4[q4][7]), "=r"(r4[q4][8]), "=r"(r4[q4][9]), "=r"(r4[q4][10]),
                          "=r"(r4[q4][11]), "=r"(r4[q4][12]), "=r"(r4[q4][13]), "=r"(r4[q4][14]), "=r"(r4[q4][15])
                        : "r"(lane_addr + kColO + c64 + q4 * 16)
                        : "memory");
                }
            }
            tc::tmem_ld_wait();
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int c0 = c64 + q4 * 16;
                if (c0 >= P.dv) continue;
                const uint32_t(&r)[16] = r4[q4];
                if (final_rows) {
                    if (!store) continue;
#pragma unroll
                    for (int j = 0; j < 16; j += 8) {
                        if (c0 + j < P.head_dim) {            // head_dim is a multiple of 8
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(r[j + 2 * e]) * inv,
                                                                                __uint_as_float(r[j + 2 * e + 1]) * inv);
                                w[e] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(o + c0 + j) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        const int ch = (c0 + j) >> 2;
                        *reinterpret_cast<uint4*>(srow + ((ch ^ (row & 7)) << 4)) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
                    }
                }
            }
        }
    }
    fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();
    if (threadIdx.x == 0 && ok && !final_rows) {
        const uint32_t bytes = static_cast<uint32_t>(kRows) * P.dvp * 4;
        bulk_store_s2g(P.part_o + tile * kRows * P.dvp, sKV, bytes);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // shared memory stays valid until the copy is done
    }
    if (warp == 1) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem, kTmemColsAttn);
    }
}

// out[row] = sum_j w_j O_j / sum_j w_j l_j with w_j = 2^(m_j - max_j m_j): one thread per 8 output columns
__global__ void __launch_bounds__(256) attention_combine_kernel(const __grid_constant__ AttnParams P, int groups) {
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int c8 = P.head_dim >> 3;
    const long long total = static_cast<long long>(groups) * P.n_rows * c8;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int c = static_cast<int>(idx % c8);
    const long long gr = idx / c8;
    const int grow = static_cast<int>(gr % P.n_rows);
    const int g = static_cast<int>(gr / P.n_rows);
    const int ga = g / P.groups_inner, gb = g - ga * P.groups_inner;
    const int rt = grow / kRows, row = grow - rt * kRows;
    const size_t tile0 = (static_cast<size_t>(g) * P.row_tiles + rt) * P.key_tiles;
    float mmax = kFloor2;
    for (int j = 0; j < P.key_tiles; ++j) mmax = fmaxf(mmax, P.part_ml[((tile0 + j) * kRows + row) * 2]);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float lsum = 0.0f;
    const int sw = row & 7;
    for (int j = 0; j < P.key_tiles; ++j) {
        const float* ml = P.part_ml + ((tile0 + j) * kRows + row) * 2;
        const float w = ex2(ml[0] - mmax);
        lsum = fmaf(w, ml[1], lsum);
        const float4* po = reinterpret_cast<const float4*>(P.part_o + ((tile0 + j) * kRows + row) * P.dvp);
        const float4 a = po[(2 * c) ^ sw], b = po[(2 * c + 1) ^ sw];
        acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]); acc[2] = fmaf(w, a.z, acc[2]); acc[3] = fmaf(w, a.w, acc[3]);
        acc[4] = fmaf(w, b.x, acc[4]); acc[5] = fmaf(w, b.y, acc[5]); acc[6] = fmaf(w, b.z, acc[6]); acc[7] = fmaf(w, b.w, acc[7]);
    }
    const float inv = 1.0f / lsum;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
        w[e] = *reinterpret_cast<const uint32_t*>(&b);
    }
    __nv_bfloat16* o = P.out + ga * P.o_stride[0] + gb * P.o_stride[1] + static_cast<size_t>(grow) * P.ldo + c * 8;
    *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
}

// The merge of attention_combine_kernel for ONE token per CTA (rows_per_token consecutive rows, one thread per
// 8 output columns), followed by what the row kernel's plain mode would do with that token's row of
// K = rows_per_token * head_dim bf16 values: row maximum -> power-of-two pre-scale into [1024, 2048) -> residual
// e2m1 pieces with UE4M3 block scales, written into the tiled A image of the next GEMM.  A 16-element block is
// shared by two adjacent threads.  Same arithmetic, bit for bit, as merge + bf16 store + row kernel.
__global__ void __launch_bounds__(1024) attention_combine_quant_kernel(const __grid_constant__ AttnParams P) {
    __shared__ float red[32];
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int c8 = P.head_dim >> 3;
    const int token = blockIdx.x;
    const int rin = threadIdx.x / c8, c = threadIdx.x - rin * c8;
    const int grow = token * P.qa_rows_per_token + rin;
    const int rt = grow / kRows, row = grow - rt * kRows;
    const size_t tile0 = static_cast<size_t>(rt) * P.key_tiles;
    float mmax = kFloor2;
    for (int j = 0; j < P.key_tiles; ++j) mmax = fmaxf(mmax, P.part_ml[((tile0 + j) * kRows + row) * 2]);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float lsum = 0.0f;
    const int sw = row & 7;
    for (int j = 0; j < P.key_tiles; ++j) {
        const float* ml = P.part_ml + ((tile0 + j) * kRows + row) * 2;
        const float w = ex2(ml[0] - mmax);
        lsum = fmaf(w, ml[1], lsum);
        const float4* po = reinterpret_cast<const float4*>(P.part_o + ((tile0 + j) * kRows + row) * P.dvp);
        const float4 a = po[(2 * c) ^ sw], b = po[(2 * c + 1) ^ sw];
        acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]); acc[2] = fmaf(w, a.z, acc[2]); acc[3] = fmaf(w, a.w, acc[3]);
        acc[4] = fmaf(w, b.x, acc[4]); acc[5] = fmaf(w, b.y, acc[5]); acc[6] = fmaf(w, b.z, acc[6]); acc[7] = fmaf(w, b.w, acc[7]);
    }
    const float inv = 1.0f / lsum;
    uint32_t w[4];
    float r[8];
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2 * e] * inv, acc[2 * e + 1] * inv);
        w[e] = *reinterpret_cast<const uint32_t*>(&b);
        r[2 * e] = __bfloat162float(b.x);            // the quantiser sees the bf16 values a reader of `out` would
        r[2 * e + 1] = __bfloat162float(b.y);
        amax = fmaxf(amax, fmaxf(fabsf(r[2 * e]), fabsf(r[2 * e + 1])));
    }
    if (P.out != nullptr) {
        __nv_bfloat16* o = P.out + static_cast<size_t>(grow) * P.ldo + c * 8;
        *reinterpret_cast<uint4*>(o) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    // the token's maximum over the whole CTA
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) amax = fmaxf(amax, red[i]);
    const int e = prescale_exponent(amax);
    const float pre = ldexpf(1.0f, e);
    if (threadIdx.x == 0) P.qa_row_scale[token] = ldexpf(1.0f, -e);
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] *= pre;
    // block (token / 128, kb / 16) of the image: [piece][128 rows][128 B, 16-byte chunks XOR-swizzled by row & 7],
    // then [piece][4 atoms of 512 B]; this thread holds half `hb` of 16-element block kb of the token's row
    const int kb = threadIdx.x >> 1, hb = threadIdx.x & 1;
    const int kb_blocks = (P.qa_rows_per_token * P.head_dim) >> 8;       // 256-wide K stages of the row
    const int rr = token & 127, jj = kb & 15;
    uint8_t* blk = P.qa_image + (static_cast<size_t>(token >> 7) * kb_blocks + (kb >> 4)) * (static_cast<size_t>(P.qa_pieces) * 18432);
    for (int p = 0; p < P.qa_pieces; ++p) {
        uint32_t word;
        const uint8_t code = quantize_half8_piece(r, word);
        if (P.qa_sf != nullptr) {
            // row-major form: piece p of the token is row p * piece_rows + token; atoms of 128 rows x 4 blocks
            const int prow = p * P.qa_piece_rows + token;
            *reinterpret_cast<uint32_t*>(P.qa_image + static_cast<size_t>(prow) * P.qa_pitch + kb * 8 + hb * 4) = word;
            if (hb == 0) {
                P.qa_sf[(static_cast<size_t>(prow >> 7) * (kb_blocks * 4) + (kb >> 2)) * 512 + (prow & 31) * 16 +
                        ((prow >> 5) & 3) * 4 + (kb & 3)] = code;
            }
            continue;
        }
        uint8_t* code_dst = blk + p * 16384 + rr * 128 + (((jj >> 1) ^ (rr & 7)) << 4) + (jj & 1) * 8 + hb * 4;
        *reinterpret_cast<uint32_t*>(code_dst) = word;
        if (hb == 0) blk[P.qa_pieces * 16384 + p * 2048 + (jj >> 2) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (jj & 3)] = code;
    }
}

}  // namespace

int device_error_attention(int clear) { return read_device_error(clear); }

}  // namespace tpb

namespace {

struct AttnDims {
    int row_tiles, key_tiles, keys_per_cta, dpad, dv, dvp, groups;
    size_t part_o_floats, part_ml_floats;
};

int attn_dims(int n_rows, int n_keys, int head_dim, int groups, AttnDims& d) {
    TPB_REQUIRE(n_rows >= 1 && n_keys >= 1 && groups >= 1, TPB200_ERR_SHAPE);
    TPB_REQUIRE(head_dim >= 8 && head_dim <= 256 && head_dim % 8 == 0, TPB200_ERR_SHAPE);
    d.row_tiles = (n_rows + 127) / 128;
    // 256 keys per CTA halve the partial results; a problem with few row tiles (the action expert: 4) is a
    // chain of latencies instead, and a CTA that loads Q + 128 keys of K and V (192 KB through its SM's L2
    // port) is done sooner than one that loads Q + 256 (320 KB)
    d.keys_per_cta = (static_cast<long long>(groups) * d.row_tiles * ((n_keys + 255) / 256) < 64 && n_keys > 128) ? 128 : 256;
    d.key_tiles = (n_keys + d.keys_per_cta - 1) / d.keys_per_cta;
    d.dpad = (head_dim + 63) / 64 * 64;
    d.dv = (head_dim + 15) / 16 * 16;
    d.dvp = (head_dim + 31) / 32 * 32;
    d.groups = groups;
    TPB_REQUIRE(d.key_tiles <= 65535 && groups <= 65535, TPB200_ERR_SHAPE);
    const size_t tiles = static_cast<size_t>(groups) * d.row_tiles * d.key_tiles;
    d.part_o_floats = tiles * 128 * d.dvp;      // unused by a launch with one key tile and no fused quantiser
    d.part_ml_floats = tiles * 128 * 2;
    return TPB200_OK;
}

// Tensor map of one operand: [outer groups][inner groups][rows][head_dim] with element strides (stride[0],
// stride[1], ld, 1).  The three outer dimensions go into the map by ascending stride; a group dimension
// with stride 0 (every group reads the same rows) becomes a dimension of size 1 whose coordinate stays 0.
bool attn_operand(tpb::AttnOperand& op, const void* base, int head_dim, int rows, long long ld, int groups_inner,
                  long long stride_inner, int groups_outer, long long stride_outer) {
    struct Dim { uint64_t size, stride_bytes; int role; };
    Dim dims[3] = {{static_cast<uint64_t>(rows), static_cast<uint64_t>(ld) * 2, 0},
                   {static_cast<uint64_t>(groups_inner), static_cast<uint64_t>(stride_inner) * 2, 1},
                   {static_cast<uint64_t>(groups_outer), static_cast<uint64_t>(stride_outer) * 2, 2}};
    for (int i = 0; i < 3; ++i) op.mul[i] = 1;
    for (int i = 1; i < 3; ++i) {
        if (dims[i].size == 1 || dims[i].stride_bytes == 0) {
            dims[i].size = 1;
            dims[i].stride_bytes = 0;                    // placed last, stride chosen below
            op.mul[i] = 0;
        }
    }
    // order: real dimensions by ascending stride, then the size-1 ones
    int order[3] = {0, 1, 2};
    std::sort(order, order + 3, [&](int a, int b) {
        const bool ua = dims[a].stride_bytes == 0, ub = dims[b].stride_bytes == 0;
        if (ua != ub) return ub;
        if (dims[a].stride_bytes != dims[b].stride_bytes) return dims[a].stride_bytes < dims[b].stride_bytes;
        return a < b;
    });
    uint64_t gdims[4] = {static_cast<uint64_t>(head_dim), 0, 0, 0};
    uint64_t strides[3];
    uint32_t box[4] = {64, 1, 1, 1};
    uint64_t span = 0;
    for (int pos = 0; pos < 3; ++pos) {
        const Dim& dm = dims[order[pos]];
        uint64_t st = dm.stride_bytes;
        if (st == 0) st = std::max<uint64_t>(span, 16);
        gdims[pos + 1] = dm.size;
        strides[pos] = st;
        span = std::max(span, (st * dm.size + 15) / 16 * 16);
        op.slot[dm.role] = pos + 1;
        if (dm.role == 0) box[pos + 1] = 128;
    }
    return tpb::make_tensor_map_bf16_nd_sw128(&op.map, base, 4, gdims, strides, box);
}

}  // namespace

extern "C" size_t tpb200_attention_workspace_size(int n_rows, int n_keys, int head_dim, int groups) {
    AttnDims d;
    if (attn_dims(n_rows, n_keys, head_dim, groups, d) != TPB200_OK) return 0;
    return (d.part_o_floats + d.part_ml_floats) * sizeof(float) + 256;
}

extern "C" int tpb200_attention(const tpb200_attention_args* a, tpb200_stream_t stream) {
    TPB_REQUIRE(a != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(a->q && a->k && a->v, TPB200_ERR_NULL);
    const bool quant = a->quant_image != nullptr;
    TPB_REQUIRE(a->out != nullptr || quant, TPB200_ERR_NULL);
    TPB_REQUIRE((a->flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    TPB_REQUIRE(a->groups_outer >= 1 && a->groups_inner >= 1, TPB200_ERR_SHAPE);
    AttnDims d;
    const int st = attn_dims(a->n_rows, a->n_keys, a->head_dim, a->groups_outer * a->groups_inner, d);
    if (st != TPB200_OK) return st;
    TPB_REQUIRE(a->ldq >= a->head_dim && a->ldk >= a->head_dim && a->ldv >= a->head_dim && a->ldo >= a->head_dim,
                TPB200_ERR_SHAPE);
    // every row and every group offset must keep 16-byte alignment (8 bf16)
    TPB_REQUIRE(tpb_aligned16(a->q) && tpb_aligned16(a->k) && tpb_aligned16(a->v) && tpb_aligned16(a->out), TPB200_ERR_ALIGN);
    TPB_REQUIRE(a->ldq % 8 == 0 && a->ldk % 8 == 0 && a->ldv % 8 == 0 && a->ldo % 8 == 0, TPB200_ERR_ALIGN);
    for (int i = 0; i < 2; ++i) {
        TPB_REQUIRE(a->q_stride[i] % 8 == 0 && a->k_stride[i] % 8 == 0 && a->v_stride[i] % 8 == 0 && a->o_stride[i] % 8 == 0,
                    TPB200_ERR_ALIGN);
        TPB_REQUIRE(a->q_stride[i] >= 0 && a->k_stride[i] >= 0 && a->v_stride[i] >= 0 && a->o_stride[i] >= 0, TPB200_ERR_SHAPE);
    }
    if (quant) {
        // one token = rows_per_token consecutive rows = one row of the GEMM operand, K = rows_per_token * head_dim
        TPB_REQUIRE(a->groups_outer == 1 && a->groups_inner == 1, TPB200_ERR_SHAPE);
        TPB_REQUIRE(a->quant_row_scale != nullptr, TPB200_ERR_NULL);
        TPB_REQUIRE(a->quant_pieces >= 1 && a->quant_pieces <= 3, TPB200_ERR_SHAPE);
        TPB_REQUIRE(a->quant_rows_per_token >= 1 && a->n_rows % a->quant_rows_per_token == 0, TPB200_ERR_SHAPE);
        const long long K = static_cast<long long>(a->quant_rows_per_token) * a->head_dim;
        TPB_REQUIRE(K % 256 == 0 && K / 8 <= 1024, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(a->quant_image), TPB200_ERR_ALIGN);
        if (a->quant_sf != nullptr) {
            TPB_REQUIRE(a->quant_pitch >= K / 2 && a->quant_pitch % 16 == 0 && tpb_aligned16(a->quant_sf), TPB200_ERR_ALIGN);
            TPB_REQUIRE(a->quant_piece_rows % 128 == 0 && a->quant_piece_rows >= a->n_rows / a->quant_rows_per_token,
                        TPB200_ERR_SHAPE);
        }
    }
    const size_t need = (d.key_tiles > 1 || quant) ? (d.part_o_floats + d.part_ml_floats) * sizeof(float) : 0;
    if (need > 0) {
        TPB_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= need, TPB200_ERR_WORKSPACE);
        TPB_REQUIRE((reinterpret_cast<uintptr_t>(a->workspace) & 255u) == 0, TPB200_ERR_ALIGN);
    }

    tpb::AttnParams P = {};
    if (!attn_operand(P.q, a->q, a->head_dim, a->n_rows, a->ldq, a->groups_inner, a->q_stride[1], a->groups_outer,
                      a->q_stride[0]) ||
        !attn_operand(P.k, a->k, a->head_dim, a->n_keys, a->ldk, a->groups_inner, a->k_stride[1], a->groups_outer,
                      a->k_stride[0]) ||
        !attn_operand(P.v, a->v, a->head_dim, a->n_keys, a->ldv, a->groups_inner, a->v_stride[1], a->groups_outer,
                      a->v_stride[0])) {
        return TPB200_ERR_SHAPE;
    }
    P.out = static_cast<__nv_bfloat16*>(a->out);
    P.key_bias = static_cast<const __nv_bfloat16*>(a->key_bias);
    P.n_rows = a->n_rows;
    P.n_keys = a->n_keys;
    P.head_dim = a->head_dim;
    P.dpad = d.dpad;
    P.dv = d.dv;
    P.dvp = d.dvp;
    P.ldo = a->ldo;
    P.groups_inner = a->groups_inner;
    for (int i = 0; i < 2; ++i) P.o_stride[i] = a->o_stride[i];
    P.scale2 = a->scale * 1.4426950408889634f;
    P.row_tiles = d.row_tiles;
    P.key_tiles = d.key_tiles;
    P.keys_per_cta = d.keys_per_cta;
    P.part_o = static_cast<float*>(a->workspace);
    P.part_ml = P.part_o + d.part_o_floats;
    P.qa_image = static_cast<uint8_t*>(a->quant_image);
    P.qa_row_scale = a->quant_row_scale;
    P.qa_pieces = a->quant_pieces;
    P.qa_rows_per_token = a->quant_rows_per_token;
    P.qa_sf = static_cast<uint8_t*>(a->quant_sf);
    P.qa_pitch = a->quant_pitch;
    P.qa_piece_rows = a->quant_piece_rows;

    const int nchunk = d.dpad / 64;
    const size_t smem = static_cast<size_t>(std::max(nchunk, 4) + 2 * nchunk) * tpb::kChunkBytes + sizeof(tpb::AttnControl) + 1024;
    static std::atomic<uint64_t> configured{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured.load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(tpb::attention_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
            cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured.fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(d.row_tiles, d.key_tiles, d.groups);
    cfg.blockDim = dim3(tpb::kThreadsAttn, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    if (a->flags & TPB200_FLAG_PDL) {
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, tpb::attention_partial_kernel, P) != cudaSuccess) return TPB200_ERR_CUDA;
    if (quant) {
        cudaLaunchConfig_t c2 = {};
        c2.gridDim = dim3(static_cast<unsigned>(a->n_rows / a->quant_rows_per_token), 1, 1);
        c2.blockDim = dim3(static_cast<unsigned>(a->quant_rows_per_token * a->head_dim / 8), 1, 1);
        c2.stream = reinterpret_cast<cudaStream_t>(stream);
        c2.attrs = attr;
        c2.numAttrs = 1;
        if (cudaLaunchKernelEx(&c2, tpb::attention_combine_quant_kernel, P) != cudaSuccess) return TPB200_ERR_CUDA;
    } else if (d.key_tiles > 1) {
        const long long threads = static_cast<long long>(d.groups) * a->n_rows * (a->head_dim / 8);
        cudaLaunchConfig_t c2 = {};
        c2.gridDim = dim3(static_cast<unsigned>((threads + 255) / 256), 1, 1);
        c2.blockDim = dim3(256, 1, 1);
        c2.stream = reinterpret_cast<cudaStream_t>(stream);
        // the merge kernel may start while the partial kernel still runs (it waits for it in griddepcontrol.wait):
        // its launch latency hides behind the tiles' work
        c2.attrs = attr;
        c2.numAttrs = 1;
        if (cudaLaunchKernelEx(&c2, tpb::attention_combine_kernel, P, d.groups) != cudaSuccess) return TPB200_ERR_CUDA;
    }
    return TPB200_OK;
}
