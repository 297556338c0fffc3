// INT4 W4A16 GEMV for ONE token in the row-major layout ([N, K/8] words, 8 codes per word along K, code i at
// bits 4i, zero point 8; fp16 / bf16 scale per `group` weights): the benchmark's config-1 shape (16384 x 2048,
// group 128) and its relatives.  Same arithmetic as the TVM kernel it replaces
// (openpi/src/openpi/ops/w4a16_gemv.py:56-102): products in fp16, sums in fp32.
//
// The general decode kernel (gemv_rowmajor.cu) spends ~3 thread-instructions per weight and is bound by
// instruction issue.  This one is written for the single shape class where that matters most and gets to ~2.2:
//   * a lane always works on the same 32-weight chunks of a row (chunk = lane, lane + 32, ...), so the token's
//     activations for those chunks sit in registers for the whole launch, already paired the way the nibbles
//     come out of a word (code j with code j + 4);
//   * a word gives four fp16 pairs with one shift + one lop3 each ((w >> 4j) & 0x000F000F | 0x64006400 is the
//     pair (1024 + q_j, 1024 + q_{j+4})), one packed subtract takes the 1032 off, one packed FMA multiplies by
//     the activations into one of four independent accumulators;
//   * the group scale is applied once per 32 weights, in fp32.
// Row tiles of 16 rows come in through a ring of bulk copies (weights with the L2 evict-first hint: they are
// read once), two CTAs per SM.  Every wait is bounded.
#include <algorithm>

#include "common.cuh"

namespace tpb {
namespace {

constexpr int kLeanThreads = 256;
constexpr int kLeanWarps = 8;
constexpr int kLeanRows = 16;      // rows per tile: two per warp
constexpr int kLeanStages = 4;

struct LeanParams {
    const uint8_t* w;
    const void* scales;
    const void* x;
    const void* bias;
    void* out;
    int scale_dtype, x_dtype, bias_dtype, out_dtype;
    int N, K, group;
    int tiles;
};

__device__ __forceinline__ __half load_x_half(const void* x, int dtype, int k) {
    if (dtype == TPB200_F16) return static_cast<const __half*>(x)[k];
    if (dtype == TPB200_BF16) return __float2half_rn(__bfloat162float(static_cast<const __nv_bfloat16*>(x)[k]));
    return __float2half_rn(static_cast<const float*>(x)[k]);
}

template <int CH>   // 32-weight chunks per lane and row: K / 1024
__global__ void __launch_bounds__(kLeanThreads, 2) w4a16_rowmajor_lean_kernel(const __grid_constant__ LeanParams P) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int row_bytes = P.K >> 1;
    const int groups = P.K / P.group;                       // scales per row
    const int w_stage = kLeanRows * row_bytes;
    const int s_stage = kLeanRows * groups * 2;
    uint8_t* wst = smem;
    uint8_t* sst = smem + kLeanStages * w_stage;
    uint64_t* full = reinterpret_cast<uint64_t*>(sst + kLeanStages * ((s_stage + 15) & ~15));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // this CTA's contiguous range of row tiles
    const int t0 = static_cast<int>(static_cast<long long>(P.tiles) * blockIdx.x / gridDim.x);
    const int t1 = static_cast<int>(static_cast<long long>(P.tiles) * (blockIdx.x + 1) / gridDim.x);
    const int ntile = t1 - t0;

    // tile t0 + i into stage i % kLeanStages.  `part` 0 arms the barrier and copies the weights, `part` 1 copies the
    // scales: a thread that issues a bulk copy is held ~0.3 us, so the first fill goes out from eight lanes at once.
    auto request = [&](int i, int part) {
        const int s = i % kLeanStages;
        const int row0 = (t0 + i) * kLeanRows;
        const int rows = min(kLeanRows, P.N - row0);
        if (part == 0) {
            bulk_copy_g2s_hint(wst + s * w_stage, P.w + static_cast<size_t>(row0) * row_bytes, rows * row_bytes, &full[s],
                               l2_policy_evict_first());
        } else {
            bulk_copy_g2s(sst + s * ((s_stage + 15) & ~15),
                          static_cast<const uint8_t*>(P.scales) + static_cast<size_t>(row0) * groups * 2, rows * groups * 2,
                          &full[s]);
        }
    };
    auto arm = [&](int i) {
        const int rows = min(kLeanRows, P.N - (t0 + i) * kLeanRows);
        mbar_expect_tx(&full[i % kLeanStages], static_cast<uint32_t>(rows * row_bytes + rows * groups * 2));
    };
    if (warp == 0) {
        if (lane == 0) {
            for (int s = 0; s < kLeanStages; ++s) mbar_init(&full[s], 1);
            fence_mbar_init();
            for (int i = 0; i < min(ntile, kLeanStages); ++i) arm(i);
        }
        __syncwarp();
        // weights and scales never depend on the previous kernel: the first tiles go out before the wait
        if (lane < 2 * kLeanStages && (lane >> 1) < ntile) request(lane >> 1, lane & 1);
    }
    pdl_launch_dependents();
    pdl_wait_prior_grids();

    // the token's activations for this lane's chunks, paired as the nibbles of a word come out: (k + j, k + j + 4)
    __half2 xr[CH][4][4];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
        const int k0 = (lane + 32 * i) * 32;
        if (P.x_dtype == TPB200_F32) {
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    xr[i][wd][j] = __halves2half2(load_x_half(P.x, P.x_dtype, k0 + 8 * wd + j),
                                                  load_x_half(P.x, P.x_dtype, k0 + 8 * wd + j + 4));
                }
            }
        } else {
            // 32 sixteen-bit values = four 16-byte loads; (e0,e1),(e2,e3),(e4,e5),(e6,e7) -> (e0,e4),(e1,e5),(e2,e6),(e3,e7)
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(P.x) + k0);
#pragma unroll
            for (int wd = 0; wd < 4; ++wd) {
                const uint4 u = __ldg(src + wd);
                uint32_t p[4] = {u.x, u.y, u.z, u.w};
                if (P.x_dtype == TPB200_BF16) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 h = __float22half2_rn(__bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&p[e])));
                        p[e] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                }
                const uint32_t q0 = __byte_perm(p[0], p[2], 0x5410), q1 = __byte_perm(p[0], p[2], 0x7632);
                const uint32_t q2 = __byte_perm(p[1], p[3], 0x5410), q3 = __byte_perm(p[1], p[3], 0x7632);
                xr[i][wd][0] = *reinterpret_cast<const __half2*>(&q0);
                xr[i][wd][1] = *reinterpret_cast<const __half2*>(&q1);
                xr[i][wd][2] = *reinterpret_cast<const __half2*>(&q2);
                xr[i][wd][3] = *reinterpret_cast<const __half2*>(&q3);
            }
        }
    }
    __syncthreads();                  // barriers initialised

    const uint32_t k1032 = 0x64086408u;
    const __half2 h1032 = *reinterpret_cast<const __half2*>(&k1032);
    // the scale group of each of this lane's chunks: the same for every row, so the division is done once
    int grp[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) grp[c] = (lane + 32 * c) / (P.group >> 5);
    bool ok = true;
    for (int i = 0; i < ntile && ok; ++i) {
        const int s = i % kLeanStages;
        if (!mbar_wait_bounded(&full[s], (i / kLeanStages) & 1)) {
            record_error(kErrGemvFullBarrierTimeout);
            ok = false;
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        const int row0 = (t0 + i) * kLeanRows;
        const uint8_t* wt = wst + s * w_stage;
        const uint8_t* st = sst + s * ((s_stage + 15) & ~15);
#pragma unroll
        for (int rr = 0; rr < kLeanRows / kLeanWarps; ++rr) {
            const int r = warp + rr * kLeanWarps;
            const int n = row0 + r;
            if (n >= P.N) continue;                          // warp-uniform
            float total = 0.0f;
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int chunk = lane + 32 * c;
                const uint4 wv = *reinterpret_cast<const uint4*>(wt + r * row_bytes + chunk * 16);
                const uint32_t words[4] = {wv.x, wv.y, wv.z, wv.w};
                __half2 acc[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = __float2half2_rn(0.0f);
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint32_t t = ((words[wd] >> (4 * j)) & 0x000F000Fu) | 0x64006400u;
                        const __half2 q = __hsub2(*reinterpret_cast<const __half2*>(&t), h1032);
                        acc[j] = __hfma2(q, xr[c][wd][j], acc[j]);
                    }
                }
                const __half2 sum2 = __hadd2(__hadd2(acc[0], acc[1]), __hadd2(acc[2], acc[3]));
                const float2 f = __half22float2(sum2);
                const float sc = P.scale_dtype == TPB200_SCALE_F16
                                     ? __half2float(reinterpret_cast<const __half*>(st)[r * groups + grp[c]])
                                     : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(st)[r * groups + grp[c]]);
                total = fmaf(f.x + f.y, sc, total);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
            if (lane == 0) {
                if (P.bias != nullptr) total += load_as_float(P.bias, P.bias_dtype, n);
                store_from_float(P.out, P.out_dtype, n, total);
            }
        }
        __syncthreads();              // the stage is free
        if (warp == 0 && i + kLeanStages < ntile) {
            if (lane == 0) arm(i + kLeanStages);
            __syncwarp();
            if (lane < 2) request(i + kLeanStages, lane);
        }
    }
}

template <int CH>
int launch_lean(const LeanParams& P, int grid, size_t smem, int flags, cudaStream_t stream) {
    if (cudaFuncSetAttribute(w4a16_rowmajor_lean_kernel<CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kLeanThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    if (cudaLaunchKernelEx(&cfg, w4a16_rowmajor_lean_kernel<CH>, P) != cudaSuccess) return TPB200_ERR_CUDA;
    return tpb_launch_status();
}

}  // namespace

// Returns TPB200_OK after launching, a negative status on a launch failure, or +1 when the shape is outside this
// kernel's class (the caller then uses the general decode kernel).  Arguments are already validated by the caller.
int w4a16_rowmajor_lean(const void* x, int x_dtype, const void* weight_packed, const void* scales, int scale_dtype,
                        const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K, int group_size,
                        int flags, cudaStream_t stream) {
    if (M != 1 || K % 1024 != 0 || K > 4096 || group_size < 32 || group_size % 32 != 0 || K % group_size != 0 || N % 16 != 0) {
        return 1;
    }
    if (scale_dtype != TPB200_SCALE_F16 && scale_dtype != TPB200_SCALE_BF16) return 1;
    if (x == nullptr || weight_packed == nullptr || scales == nullptr || out == nullptr) return 1;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        return TPB200_ERR_CUDA;
    }
    LeanParams P;
    P.w = static_cast<const uint8_t*>(weight_packed);
    P.scales = scales;
    P.x = x;
    P.bias = bias;
    P.out = out;
    P.scale_dtype = scale_dtype;
    P.x_dtype = x_dtype;
    P.bias_dtype = bias_dtype;
    P.out_dtype = out_dtype;
    P.N = N;
    P.K = K;
    P.group = group_size;
    P.tiles = (N + kLeanRows - 1) / kLeanRows;
    const int groups = K / group_size;
    const size_t smem = static_cast<size_t>(kLeanStages) * (kLeanRows * (K / 2) + ((kLeanRows * groups * 2 + 15) & ~15)) +
                        kLeanStages * sizeof(uint64_t) + 256;
    const int grid = std::min(2 * sms, P.tiles);
    switch (K / 1024) {
        case 1: return launch_lean<1>(P, grid, smem, flags, stream);
        case 2: return launch_lean<2>(P, grid, smem, flags, stream);
        case 4: return launch_lean<4>(P, grid, smem, flags, stream);
        default: return 1;          // K = 3072: not a power-of-two chunk count per lane
    }
}

}  // namespace tpb
