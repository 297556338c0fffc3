// W4A16 GEMM for more than a handful of tokens: bf16 activations x INT4 weights on the tensor cores.
//
//   out[M, N] = alpha * x[M, K] @ dequant(W)[N, K]^T (+ beta * out)
//
// INT4 x bf16 is not an operand pair of the tensor cores, so the weights are dequantised to bf16 on the way
// into shared memory -- once per CTA and K stage, then used by the MMAs of up to two 128-row tiles of
// tokens (256 tokens x 256 output columns per CTA, two fp32 accumulators filling tensor memory).  The tile is
// as large as tensor memory allows because the activations are re-read once per 256 output columns: with
// 128-column tiles those reads (373 MB through L2 for 712 x 16384 x 2048) cost more than the MMAs.
// Two weight formats:
//   plugin   signed nibbles [N, K/2] bytes (low nibble = even k), bf16 scale and optional bf16 zero point per
//            128 along K: w = q * scale + zero          (openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:41-59)
//   packer   the reference packer's (K/32, N, 4) int32 words (nibble i of word u = k % 32 == 8 u + i),
//            fp16 scale per 32, zero point 8: w = (q - 8) * scale
//            (openpi/src/openpi/utils/w4a16_packer.py:311-368, modules/w4a16_linear.py:174-199)
//
// Roles (320 threads): warps 0..7 turn one weight row each (64 K values per stage: 32 bytes -> one 128-byte
// swizzled row of bf16) and later run the epilogue; warp 8 lane 0 requests the activation tiles by TMA
// (128 rows x 128 bytes, 128-byte swizzle, rows past M read as zero); warp 9 allocates tensor memory and its
// lane 0 issues tcgen05.mma kind::f16.  The MMAs of stage k run while the threads dequantise stage k + 1.
// Every wait is bounded; nothing waits on another CTA.
#include <algorithm>
#include <atomic>

#include "tcgen05.cuh"

namespace tpb {

bool make_tensor_map_bytes_sw128(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                                 uint64_t pitch_bytes, uint32_t box_rows);

namespace {

constexpr int kTileN = 256;            // output columns per CTA
constexpr int kTileM = 128;            // token rows per accumulator
constexpr int kMaxMt = 2;              // accumulators per CTA
constexpr int kStageK = 64;            // K values per stage: one 128-byte row of bf16
constexpr int kChunk = 128 * 128;      // bytes of one 128-row operand tile of a stage
constexpr int kBTile = kTileN * 128;   // bytes of the dequantised weight tile of a stage
constexpr int kAStages = 3, kBStages = 2;
constexpr int kDequantThreads = kTileN;
constexpr int kThreadsW4 = kDequantThreads + 64;
constexpr int kTmaWarp = kDequantThreads / 32, kMmaWarp = kTmaWarp + 1;
constexpr long long kWaitW4 = 400000000LL;   // ~0.2 s

struct W4Params {
    CUtensorMap map_x;                 // activations as bytes [M, 2 K]
    const uint8_t* w;                  // plugin: [N, K/2] bytes; packer: (K/32, N, 4) int32
    const void* scale;                 // plugin: bf16 [N, K/128]; packer: fp16 [K/32, N]
    const __nv_bfloat16* zero;         // plugin only, may be null
    const void* bias;                  // optional, bias_dtype, added after alpha
    void* out;
    int bias_dtype, out_dtype;
    int M, N, K, ldo;
    float alpha, beta;
    int mt_per_cta;                    // 1 or 2 token tiles per CTA
    int m_tiles;
};

struct W4Control {
    uint64_t a_full[kAStages], a_empty[kAStages], b_full[kBStages], b_empty[kBStages], acc_full;
    uint32_t tmem_base;
};

__host__ __device__ constexpr uint32_t idesc_bf16_kmajor(int n) {
    // kind::f16: D = f32 ([4,6) = 1), A = B = bf16 ([7,10) = [10,13) = 1), both K-major, N >> 3 at [17,23), M >> 4 at [24,29)
    return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
        : "memory");
}

// 8 nibbles of one word (nibble i at bits 4 i) -> 8 bf16 of q * scale + zero, as one 16-byte chunk.
// `flip` = 0x88888888 for two's-complement nibbles (q = ((nib ^ 8) - 8)), 0 for unsigned nibbles with zero point 8.
__device__ __forceinline__ uint4 dequant8(uint32_t w, uint32_t flip, float scale, float zero) {
    w ^= flip;
    float f[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        // (1024 + u_j, 1024 + u_{j+4}) as exact fp16, minus 1032 -> (q_j, q_{j+4})
        uint32_t t = ((w >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
        const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&t), __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408)));
        const float2 q = __half22float2(h);
        f[j] = fmaf(q.x, scale, zero);
        f[j + 4] = fmaf(q.y, scale, zero);
    }
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
        o[j] = *reinterpret_cast<const uint32_t*>(&b);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}

template <bool kPacker>
__global__ void __launch_bounds__(kThreadsW4, 1) w4a16_gemm_tc_kernel(const __grid_constant__ W4Params P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sA = smem;                                            // [kAStages][kMaxMt][16 KB]
    uint8_t* sB = sA + kAStages * kMaxMt * kChunk;                 // [kBStages][32 KB]
    W4Control* ctl = reinterpret_cast<W4Control*>(sB + kBStages * kBTile);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kTileN;
    const int mt0 = blockIdx.y * P.mt_per_cta;
    const int nmt = min(P.mt_per_cta, P.m_tiles - mt0);
    const int nks = P.K / kStageK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(&ctl->a_full[s], 1);
            mbar_init(&ctl->a_empty[s], 1);
        }
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(&ctl->b_full[s], kDequantThreads);
            mbar_init(&ctl->b_empty[s], 1);
        }
        mbar_init(&ctl->acc_full, 1);
        fence_mbar_init();
    }
    if (warp == kMmaWarp) {
        __syncwarp();
        tc::tmem_alloc(&ctl->tmem_base, 512);
        tc::tmem_relinquish();
    }
    if (warp == kTmaWarp && lane == 0) tc::prefetch_tensormap(&P.map_x);
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem = ctl->tmem_base;
    pdl_launch_dependents();

    bool ok = true;
    if (warp == kTmaWarp) {
        // ------------------------------------------------------------ activation tiles by TMA
        if (lane == 0) {
            pdl_wait_prior_grids();
            for (int ks = 0; ks < nks; ++ks) {
                const int s = ks % kAStages;
                if (ks >= kAStages && !mbar_wait_bounded(&ctl->a_empty[s], ((ks / kAStages) - 1) & 1, kWaitW4)) {
                    record_error(kErrGemmEmptyBarrierTimeout);
                    break;
                }
                mbar_expect_tx(&ctl->a_full[s], static_cast<uint32_t>(nmt) * kChunk);
                for (int t = 0; t < nmt; ++t) {
                    tc::tma_load_2d(sA + (s * kMaxMt + t) * kChunk, &P.map_x, ks * 128, (mt0 + t) * kTileM, &ctl->a_full[s]);
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = idesc_bf16_kmajor(kTileN);
            const uint32_t a16 = smem_u32(sA) >> 4, b16 = smem_u32(sB) >> 4;
            for (int ks = 0; ks < nks; ++ks) {
                const int sa = ks % kAStages, sb = ks % kBStages;
                if (!mbar_wait_bounded(&ctl->a_full[sa], (ks / kAStages) & 1, kWaitW4) ||
                    !mbar_wait_bounded(&ctl->b_full[sb], (ks / kBStages) & 1, kWaitW4)) {
                    record_error(kErrGemmTmaBarrierTimeout);
                    break;
                }
                tc::fence_after_thread_sync();
#pragma unroll
                for (int kk = 0; kk < kStageK / 16; ++kk) {
                    const uint64_t bdesc = tc::desc_from_words(b16 + ((sb * kBTile + kk * 32) >> 4), tc::kDescHiKmajorSw128);
                    for (int t = 0; t < nmt; ++t) {
                        mma_bf16_ss(tmem + t * kTileN,
                                    tc::desc_from_words(a16 + (((sa * kMaxMt + t) * kChunk + kk * 32) >> 4), tc::kDescHiKmajorSw128),
                                    bdesc, idesc, (ks > 0 || kk > 0) ? 1u : 0u);
                    }
                }
                tc::commit(&ctl->a_empty[sa]);
                tc::commit(&ctl->b_empty[sb]);
            }
            tc::commit(&ctl->acc_full);
        }
    } else {
        // ------------------------------------------------------------ weight rows: dequantise into shared memory
        const int r = threadIdx.x;                       // 0..255: row of the weight tile = output column n0 + r
        const int n = n0 + r;
        const bool row_ok = n < P.N;
        const uint32_t flip = kPacker ? 0u : 0x88888888u;
        uint4 raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
        float nsc[2] = {0.0f, 0.0f}, nzp[2] = {0.0f, 0.0f};
        // codes AND scales of a stage are requested one stage ahead: a scale fetched at the moment it is needed
        // costs a memory round trip per stage, more than the stage's arithmetic
        auto load_raw = [&](int ks) {
            if (!row_ok) return;
            if (kPacker) {
                // (K/32, N, 4) words: the stage's two 32-blocks of this row
                const uint4* w = reinterpret_cast<const uint4*>(P.w);
                raw[0] = __ldg(w + static_cast<size_t>(2 * ks) * P.N + n);
                raw[1] = __ldg(w + static_cast<size_t>(2 * ks + 1) * P.N + n);
                const __half* sp = static_cast<const __half*>(P.scale);
                nsc[0] = __half2float(__ldg(sp + static_cast<size_t>(2 * ks) * P.N + n));
                nsc[1] = __half2float(__ldg(sp + static_cast<size_t>(2 * ks + 1) * P.N + n));
            } else {
                const uint4* w = reinterpret_cast<const uint4*>(P.w + static_cast<size_t>(n) * (P.K / 2) + ks * 32);
                raw[0] = __ldg(w);
                raw[1] = __ldg(w + 1);
                const size_t gi = static_cast<size_t>(n) * (P.K / 128) + (ks >> 1);      // 128 along K = two stages
                nsc[0] = nsc[1] = __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(P.scale) + gi));
                if (P.zero != nullptr) nzp[0] = nzp[1] = __bfloat162float(__ldg(P.zero + gi));
            }
        };
        load_raw(0);
        for (int ks = 0; ks < nks && ok; ++ks) {
            const int sb = ks % kBStages;
            const float sc[2] = {nsc[0], nsc[1]}, zp[2] = {nzp[0], nzp[1]};
            const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
            if (ks + 1 < nks) load_raw(ks + 1);          // the next stage's bytes travel during this stage's arithmetic
            if (ks >= kBStages && !mbar_wait_bounded(&ctl->b_empty[sb], ((ks / kBStages) - 1) & 1, kWaitW4)) {
                record_error(kErrGemmEmptyBarrierTimeout);
                ok = false;
                break;
            }
            uint8_t* row = sB + sb * kBTile + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint4 v = dequant8(w[c], flip, sc[c >> 2], zp[c >> 2]);
                *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) = v;
            }
            fence_proxy_async_smem();
            mbar_arrive(&ctl->b_full[sb]);
        }
        // ------------------------------------------------------------ epilogue: thread = token row of each accumulator
        if (ok && !mbar_wait_bounded(&ctl->acc_full, 0, kWaitW4)) {
            record_error(kErrGemmMmaBarrierTimeout);
            ok = false;
        }
        ok = __all_sync(0xffffffffu, ok);                // the tensor-memory loads are warp-collective
        tc::fence_after_thread_sync();
        if (ok) {
            // warps 0..3 take the accumulators' columns [0, 128), warps 4..7 columns [128, 256); the warp's
            // quarter of the 128 token rows (tensor-memory lanes) is warp % 4
            const int tr = threadIdx.x & 127;
            const int col_half = threadIdx.x >> 7;
            const uint32_t lane_addr = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16);
            for (int t = 0; t < nmt; ++t) {
                const int m = (mt0 + t) * kTileM + tr;
                const bool store = m < P.M;
                for (int c0 = col_half * 128; c0 < col_half * 128 + 128; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_32x32b_x32(lane_addr + t * kTileN + c0, v);
                    tc::tmem_ld_wait();
                    if (!store) continue;
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
                        const int nn = n0 + c0 + j;
                        if (nn >= P.N) continue;         // N is a multiple of 8
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            f[e] = __uint_as_float(v[j + e]) * P.alpha;
                            if (P.bias != nullptr) f[e] += load_as_float(P.bias, P.bias_dtype, nn + e);
                        }
                        const size_t o = static_cast<size_t>(m) * P.ldo + nn;
                        if (P.out_dtype == TPB200_BF16) {
                            __nv_bfloat16* op = static_cast<__nv_bfloat16*>(P.out) + o;
                            if (P.beta != 0.0f) {
                                const uint4 old = *reinterpret_cast<const uint4*>(op);
                                const uint32_t ow[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 p2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&ow[e]));
                                    f[2 * e] = fmaf(P.beta, p2.x, f[2 * e]);
                                    f[2 * e + 1] = fmaf(P.beta, p2.y, f[2 * e + 1]);
                                }
                            }
                            uint32_t pw[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 b2 = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
                                pw[e] = *reinterpret_cast<const uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(op) = make_uint4(pw[0], pw[1], pw[2], pw[3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                if (P.beta != 0.0f) f[e] = fmaf(P.beta, load_as_float(P.out, P.out_dtype, o + e), f[e]);
                                store_from_float(P.out, P.out_dtype, o + e, f[e]);
                            }
                        }
                    }
                }
            }
        }
    }

    tc::fence_before_thread_sync();
    __syncthreads();
    if (warp == kMmaWarp) {
        tc::fence_after_thread_sync();
        tc::tmem_dealloc(tmem, 512);
    }
}

}  // namespace

int device_error_w4a16_gemm_tc(int clear) { return read_device_error(clear); }

// format 0 = plugin (signed nibbles, bf16 scale / zero per 128), 1 = packer ((K/32, N, 4) words, fp16 scale per 32)
int w4a16_gemm_tc_launch(int format, const void* x, const void* w, const void* scale, const void* zero, const void* bias,
                         int bias_dtype, void* out, int out_dtype, int M, int N, int K, int ldo, float alpha, float beta,
                         int flags, cudaStream_t stream) {
    TPB_REQUIRE(x && w && scale && out, TPB200_ERR_NULL);
    TPB_REQUIRE(M >= 1 && N >= 8 && N % 8 == 0 && K >= 128 && K % 128 == 0 && ldo >= N, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_aligned16(x) && tpb_aligned16(w) && tpb_aligned16(out), TPB200_ERR_ALIGN);
    TPB_REQUIRE((static_cast<long long>(ldo) * tpb_dtype_size(out_dtype)) % 16 == 0, TPB200_ERR_ALIGN);
    TPB_REQUIRE(tpb_valid_dtype(out_dtype) && tpb_valid_dtype(bias_dtype), TPB200_ERR_ENUM);
    TPB_REQUIRE(format == 0 || (format == 1 && zero == nullptr), TPB200_ERR_ENUM);
    W4Params P = {};
    if (!make_tensor_map_bytes_sw128(&P.map_x, x, static_cast<uint64_t>(K) * 2, M, static_cast<uint64_t>(K) * 2, kTileM)) {
        return TPB200_ERR_CUDA;
    }
    P.w = static_cast<const uint8_t*>(w);
    P.scale = scale;
    P.zero = static_cast<const __nv_bfloat16*>(zero);
    P.bias = bias;
    P.out = out;
    P.bias_dtype = bias_dtype;
    P.out_dtype = out_dtype;
    P.M = M;
    P.N = N;
    P.K = K;
    P.ldo = ldo;
    P.alpha = alpha;
    P.beta = beta;
    P.m_tiles = (M + kTileM - 1) / kTileM;
    // two token tiles per CTA halve the weight reads and dequantisations; with too few CTAs for the machine
    // one tile per CTA doubles the CTAs instead
    int sms = 148;
    {
        int dev_ = 0;
        if (cudaGetDevice(&dev_) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_);
    }
    const int n_tiles = (N + kTileN - 1) / kTileN;
    P.mt_per_cta = (P.m_tiles > 1 && n_tiles * ((P.m_tiles + 1) / 2) >= sms) ? 2 : 1;
    const int m_groups = (P.m_tiles + P.mt_per_cta - 1) / P.mt_per_cta;
    const size_t smem = static_cast<size_t>(kAStages * kMaxMt) * kChunk + static_cast<size_t>(kBStages) * kBTile +
                        sizeof(W4Control) + 1024;
    auto kernel = format == 1 ? w4a16_gemm_tc_kernel<true> : w4a16_gemm_tc_kernel<false>;
    static std::atomic<uint64_t> configured[2] = {{0}, {0}};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(configured[format].load(std::memory_order_relaxed) & bit)) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
        configured[format].fetch_or(bit, std::memory_order_relaxed);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, m_groups, 1);
    cfg.blockDim = dim3(kThreadsW4, 1, 1);
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

}  // namespace tpb

extern "C" int tpb200_w4a16_gemm(const void* x, const void* weight, const void* scales, const void* zeros,
                                 const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K, int ldo,
                                 int layout, float alpha, float beta, int flags, tpb200_stream_t stream) {
    TPB_REQUIRE((flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    TPB_REQUIRE(layout == TPB200_INT4_KBLOCK || layout == TPB200_INT4_PLUGIN, TPB200_ERR_ENUM);
    return tpb::w4a16_gemm_tc_launch(layout == TPB200_INT4_KBLOCK ? 1 : 0, x, weight, scales, zeros, bias, bias_dtype, out,
                                     out_dtype, M, N, K, ldo == 0 ? N : ldo, alpha, beta, flags,
                                     reinterpret_cast<cudaStream_t>(stream));
}
