// The GEMM launchers of the reference's TensorRT plugins, with their names and signatures:
//   w4a16GemmForward / getW4A16GemmWorkspaceSize   openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:41-59
//   w4a8GemmForward  / getW4A8GemmWorkspaceSize    openpi/w4a8_plugin/src/w4a8_gemm_plugin.h:39-57
// Both are thin host compositions of the library's kernels; everything they need beyond inputs
// and outputs lives in the caller's workspace.
#include <algorithm>

#include "common.cuh"

namespace tpb {
int w4a16_gemm_tc_launch(int format, const void* x, const void* w, const void* scale, const void* zero, const void* bias,
                         int bias_dtype, void* out, int out_dtype, int M, int N, int K, int ldo, float alpha, float beta,
                         int flags, cudaStream_t stream);
}

namespace tpb {

int gemv_rowmajor_single(int fmt_is_u4, const void* x, int x_dtype, const void* x_scales, const void* w,
                         const void* scales, int scale_dtype, int group, float global_scale, const void* bias,
                         int bias_dtype, void* out, int out_dtype, int M, int N, int K, int activation, int flags,
                         cudaStream_t stream);
void set_last_error(int status);

namespace {

constexpr int kW4A16Group = 128;   // W4A16_GROUP_SIZE, w4a16_gemm_plugin.h:37

// xsum[m, g] = sum of x[m, k] over group g (for the zero-point term)
__global__ void group_sums_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ xsum, int M, int K, int group) {
    const int G = K / group;
    const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);    // one warp per (m, g)
    if (idx >= M * G) return;
    const int m = idx / G, g = idx % G;
    float s = 0.0f;
    for (int k = threadIdx.x & 31; k < group; k += 32) s += __bfloat162float(x[static_cast<size_t>(m) * K + g * group + k]);
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) xsum[idx] = s;
}

// out = acc + alpha * sum_g zero[n, g] * xsum[m, g] + beta * out
__global__ void w4a16_epilogue_kernel(const float* __restrict__ acc, const float* __restrict__ xsum,
                                      const __nv_bfloat16* __restrict__ zeros, __nv_bfloat16* __restrict__ out, int M,
                                      int N, int G, float alpha, float beta) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(M) * N) return;
    const int m = static_cast<int>(t / N), n = static_cast<int>(t % N);
    float v = acc[t];
    if (zeros != nullptr) {
        float z = 0.0f;
        for (int g = 0; g < G; ++g) z = fmaf(__bfloat162float(zeros[static_cast<size_t>(n) * G + g]), xsum[m * G + g], z);
        v = fmaf(alpha, z, v);
    }
    if (beta != 0.0f) v = fmaf(beta, __bfloat162float(out[t]), v);
    out[t] = __float2bfloat16_rn(v);
}

}  // namespace
}  // namespace tpb

extern "C" size_t getW4A16GemmWorkspaceSize(int M, int N, int K) {
    if (M < 1 || N < 1 || K < tpb::kW4A16Group) return 0;
    // fp32 accumulators [M, N] + group sums [M, K / 128]; only touched when zero points or beta are in use
    return (static_cast<size_t>(M) * N + static_cast<size_t>(M) * (K / tpb::kW4A16Group)) * sizeof(float) + 256;
}

extern "C" void w4a16GemmForward(const void* activation, const void* weight_packed, const void* weight_scale,
                                 const void* weight_zero, void* output, int M, int N, int K, float alpha, float beta,
                                 void* workspace, size_t workspaceSize, tpb200_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    const int G = K / tpb::kW4A16Group;
    if (!activation || !weight_packed || !weight_scale || !output) return tpb::set_last_error(TPB200_ERR_NULL);
    if (M < 1 || N < 1 || K < tpb::kW4A16Group || K % tpb::kW4A16Group != 0) return tpb::set_last_error(TPB200_ERR_SHAPE);
    if (M > 16) {
        // prefill-sized: one tensor-core launch (zero points, alpha and beta in its epilogue; no workspace)
        const int st = tpb::w4a16_gemm_tc_launch(0, activation, weight_packed, weight_scale, weight_zero, nullptr, TPB200_F32,
                                                 output, TPB200_BF16, M, N, K, N, alpha, beta, TPB200_FLAG_NONE, stream);
        tpb::set_last_error(st);
        return;
    }
    const bool extra = (weight_zero != nullptr) || (beta != 0.0f);
    float* acc = nullptr;
    float* xsum = nullptr;
    if (extra) {
        if (workspace == nullptr || workspaceSize < getW4A16GemmWorkspaceSize(M, N, K) ||
            (reinterpret_cast<uintptr_t>(workspace) & 15u)) {
            return tpb::set_last_error(TPB200_ERR_WORKSPACE);
        }
        acc = static_cast<float*>(workspace);
        xsum = acc + static_cast<size_t>(M) * N;
    }
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(activation);
    // the decode kernel takes up to 16 rows per launch
    for (int m0 = 0; m0 < M; m0 += 16) {
        const int mc = std::min(16, M - m0);
        void* dst = extra ? static_cast<void*>(acc + static_cast<size_t>(m0) * N)
                          : static_cast<void*>(static_cast<__nv_bfloat16*>(output) + static_cast<size_t>(m0) * N);
        const int st = tpb::gemv_rowmajor_single(2, x + static_cast<size_t>(m0) * K, TPB200_BF16, nullptr, weight_packed,
                                                 weight_scale, TPB200_SCALE_BF16, tpb::kW4A16Group, alpha, nullptr,
                                                 TPB200_F32, dst, extra ? TPB200_F32 : TPB200_BF16, mc, N, K,
                                                 TPB200_ACT_NONE, TPB200_FLAG_NONE, stream);
        if (st != TPB200_OK) return tpb::set_last_error(st);
    }
    if (extra) {
        if (weight_zero != nullptr) {
            const int warps = M * G;
            tpb::group_sums_kernel<<<(warps + 7) / 8, 256, 0, stream>>>(x, xsum, M, K, tpb::kW4A16Group);
        }
        const long long total = static_cast<long long>(M) * N;
        tpb::w4a16_epilogue_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
            acc, xsum, static_cast<const __nv_bfloat16*>(weight_zero), static_cast<__nv_bfloat16*>(output), M, N, G,
            alpha, beta);
    }
    tpb::set_last_error(tpb_launch_status());
}

// ---------------------------------------------------------------------------------------------
// w4a8GemmForward: FP8-E4M3 activations (+ E4M3 scale per 16) x e2m1 weights stored TRANSPOSED
// ([K/2, N] codes, [K/16, N] E4M3 scales).  The tensor-core kernel wants K-major operands and its own
// scale layout, so each call (1) re-lays the weights out into the workspace, (2) expands the FP8
// activations to bf16 (exact: 4 x 4 significand bits), (3) splits them into residual e2m1 pieces and
// (4) runs the block-scaled GEMM.  (The reference's kernel declares MX types with UE8M0 scales per
// 32 while its host code fills E4M3 scales per 16; the semantics implemented here are the host
// code's: value = fp8 * scale.)
// ---------------------------------------------------------------------------------------------
namespace tpb {
namespace {

struct W4A8Layout {
    size_t b_packed, b_sf, x_bf16, a_packed, a_sf, row_scale, total;
    int pitch, piece_rows;
};

constexpr int kW4A8Pieces = 3;

W4A8Layout w4a8_layout(int M, int N, int K) {
    W4A8Layout L;
    L.pitch = (K / 2 + 15) / 16 * 16;
    L.piece_rows = (M + 127) / 128 * 128;
    auto up = [](size_t v) { return (v + 255) / 256 * 256; };
    size_t off = 0;
    L.b_packed = off; off = up(off + static_cast<size_t>(N) * L.pitch);
    L.b_sf = off;     off = up(off + tpb200_nvfp4_sf_bytes(N, K));
    L.x_bf16 = off;   off = up(off + static_cast<size_t>(M) * K * 2);
    L.a_packed = off; off = up(off + static_cast<size_t>(kW4A8Pieces) * L.piece_rows * L.pitch);
    L.a_sf = off;     off = up(off + tpb200_nvfp4_sf_bytes(kW4A8Pieces * L.piece_rows, K));
    L.row_scale = off; off = up(off + static_cast<size_t>(M) * 4);
    L.total = off;
    return L;
}

// thread -> (16-block kb, column n): gathers the block's 8 code bytes from the [K/2, N] matrix and its
// scale from [K/16, N]; consecutive threads read consecutive n
__global__ void w4a8_prepare_weight_kernel(const uint8_t* __restrict__ packed_t, const uint8_t* __restrict__ scales_t,
                                           uint8_t* __restrict__ b, int pitch, uint8_t* __restrict__ b_sf, int N, int K,
                                           int rows_pad, int kb_pad) {
    const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (t >= static_cast<long long>(rows_pad) * kb_pad) return;
    const int kb = static_cast<int>(t / rows_pad);
    const int n = static_cast<int>(t % rows_pad);
    const size_t sf_off = (static_cast<size_t>(n >> 7) * (kb_pad >> 2) + (kb >> 2)) * 512 + (n & 31) * 16 +
                          ((n >> 5) & 3) * 4 + (kb & 3);
    if (n >= N || kb * 16 >= K) {
        b_sf[sf_off] = 0;
        return;
    }
    b_sf[sf_off] = scales_t[static_cast<size_t>(kb) * N + n];
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t byte = packed_t[(static_cast<size_t>(kb) * 8 + i) * N + n];
        if (i < 4) lo |= byte << (8 * i);
        else hi |= byte << (8 * (i - 4));
    }
    *reinterpret_cast<uint2*>(b + static_cast<size_t>(n) * pitch + kb * 8) = make_uint2(lo, hi);
}

__global__ void w4a8_dequant_act_kernel(const uint8_t* __restrict__ a8, const uint8_t* __restrict__ sa,
                                        __nv_bfloat16* __restrict__ x, long long nblocks) {
    const long long bidx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (bidx >= nblocks) return;
    const float s = decode_e4m3(sa[bidx]);
    const uint4 v = *reinterpret_cast<const uint4*>(a8 + bidx * 16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f0 = decode_e4m3x2(static_cast<uint16_t>(w[i] & 0xFFFF));
        const float2 f1 = decode_e4m3x2(static_cast<uint16_t>(w[i] >> 16));
        __nv_bfloat162 b0 = __floats2bfloat162_rn(f0.x * s, f0.y * s);
        __nv_bfloat162 b1 = __floats2bfloat162_rn(f1.x * s, f1.y * s);
        o[2 * i] = *reinterpret_cast<uint32_t*>(&b0);
        o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b1);
    }
    uint4* dst = reinterpret_cast<uint4*>(x + bidx * 16);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

}  // namespace
}  // namespace tpb

extern "C" size_t getW4A8GemmWorkspaceSize(int M, int N, int K) {
    if (M < 1 || N < 1 || K < 16) return 0;
    return tpb::w4a8_layout(M, N, K).total + 256;
}

extern "C" void w4a8GemmForward(const void* activation, const void* activation_scale, const void* weight_packed,
                                const void* weight_scale, void* output, int M, int N, int K, float alpha,
                                void* workspace, size_t workspaceSize, tpb200_stream_t stream_) {
    cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
    if (!activation || !activation_scale || !weight_packed || !weight_scale || !output)
        return tpb::set_last_error(TPB200_ERR_NULL);
    if (M < 1 || N < 8 || N % 8 != 0 || K < 16 || K % 16 != 0) return tpb::set_last_error(TPB200_ERR_SHAPE);
    if (workspace == nullptr || workspaceSize < getW4A8GemmWorkspaceSize(M, N, K)) return tpb::set_last_error(TPB200_ERR_WORKSPACE);
    uint8_t* ws = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(workspace) + 255) & ~uintptr_t(255));
    const tpb::W4A8Layout L = tpb::w4a8_layout(M, N, K);
    const int rows_pad = (N + 127) / 128 * 128;
    const int kb_pad = (K + 255) / 256 * 16;
    {
        const long long total = static_cast<long long>(rows_pad) * kb_pad;
        tpb::w4a8_prepare_weight_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(weight_packed), static_cast<const uint8_t*>(weight_scale), ws + L.b_packed, L.pitch,
            ws + L.b_sf, N, K, rows_pad, kb_pad);
        const long long nblocks = static_cast<long long>(M) * (K / 16);
        tpb::w4a8_dequant_act_kernel<<<static_cast<unsigned>((nblocks + 255) / 256), 256, 0, stream>>>(
            static_cast<const uint8_t*>(activation), static_cast<const uint8_t*>(activation_scale),
            reinterpret_cast<__nv_bfloat16*>(ws + L.x_bf16), nblocks);
    }
    int st = tpb200_nvfp4_quantize_act_pieces(ws + L.x_bf16, TPB200_BF16, K, ws + L.a_packed, L.pitch, ws + L.a_sf,
                                              reinterpret_cast<float*>(ws + L.row_scale), M, K, tpb::kW4A8Pieces,
                                              L.piece_rows, stream_);
    if (st != TPB200_OK) return tpb::set_last_error(st);
    tpb200_nvfp4_gemm_args a = {};
    a.a_packed = ws + L.a_packed; a.a_pitch = L.pitch; a.a_sf = ws + L.a_sf;
    a.a_pieces = tpb::kW4A8Pieces; a.a_piece_rows = L.piece_rows; a.a_row_scale = reinterpret_cast<float*>(ws + L.row_scale);
    a.b_packed = ws + L.b_packed; a.b_pitch = L.pitch; a.b_sf = ws + L.b_sf;
    a.alpha = alpha; a.activation = TPB200_ACT_NONE;
    a.out = output; a.out_dtype = TPB200_BF16; a.ldo = N;
    a.M = M; a.N = N; a.K = K;
    st = tpb200_nvfp4_gemm_ex(&a, stream_);
    tpb::set_last_error(st != TPB200_OK ? st : tpb_launch_status());
}
