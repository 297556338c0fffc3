// Row-wise glue fused with the activation quantiser of the tensor-core GEMM.
//
// Between two linears the model only does row-local work (residual add, RMSNorm / adaptive
// RMSNorm / LayerNorm, GELU(gate) * up).  Each of these is one kernel here that reads the bf16
// inputs once, does the arithmetic in fp32 with the roundings the PyTorch modules apply
// (openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:49-129,
// 212-230), and writes the result straight in the GEMM's operand format: residual e2m1 pieces +
// UE4M3 block scales + the per-row power-of-two multiplier (see nvfp4_gemm.cu).  A bf16 copy of
// the transformed row and the updated residual stream are written only when asked for.
// One CTA per row; the transformed row is staged in shared memory (K <= 16384).
#include "common.cuh"

namespace tpb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxK = 16384;

struct RowOpParams {
    int mode;
    int M, K;
    const __nv_bfloat16* x;        // main input [M, ldx] (GELU_MUL: [M, 2K] = gate | up)
    int ldx;
    // residual:  h = res_in + x * gate   (gate optional, [K]);  h_out optional
    const __nv_bfloat16* res_in;
    const __nv_bfloat16* gate;
    __nv_bfloat16* h_out;
    // norm parameters: RMS: weight [K] (1 + w) ; ADA: scale, shift [K] ; LAYERNORM: weight, bias [K]
    const __nv_bfloat16* w0;
    const __nv_bfloat16* w1;
    float eps;
    // outputs
    __nv_bfloat16* y_out;          // optional bf16 copy of the transformed row [M, K]
    uint8_t* packed;               // [pieces * piece_rows, pitch]
    int pitch;
    uint8_t* sf;                   // swizzled scales of pieces * piece_rows rows
    float* row_scale;              // [M]
    int pieces, piece_rows, kb_pad;
    int tiled;                     // packed = tiled A image of the GEMM: blocks [m / 128][k / 256] of pieces * 18 KB
};

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; ++i) t = fmaxf(t, red[i]);
    return t;
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__global__ void __launch_bounds__(kThreads) row_transform_quantize_kernel(const __grid_constant__ RowOpParams P) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* row = reinterpret_cast<float*>(smem);            // K floats: the row being transformed
    __shared__ float red[kThreads / 32];
    const int m = blockIdx.x;
    const int K = P.K;
    const int tid = threadIdx.x;

    // ---- load (+ residual) ------------------------------------------------------------------
    if (P.mode == TPB200_ROW_GELU_MUL) {
        const __nv_bfloat16* g = P.x + static_cast<size_t>(m) * P.ldx;
        const __nv_bfloat16* u = g + K;
        for (int k = tid * 2; k < K; k += kThreads * 2) {
            const float2 gv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(g + k));
            const float2 uv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(u + k));
            row[k] = bf16r(bf16r(gelu_tanh(gv.x)) * uv.x);
            row[k + 1] = bf16r(bf16r(gelu_tanh(gv.y)) * uv.y);
        }
    } else {
        const __nv_bfloat16* xr = P.x + static_cast<size_t>(m) * P.ldx;
        for (int k = tid * 2; k < K; k += kThreads * 2) {
            float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xr + k));
            if (P.res_in != nullptr) {
                const float2 h = __bfloat1622float2(
                    *reinterpret_cast<const __nv_bfloat162*>(P.res_in + static_cast<size_t>(m) * K + k));
                if (P.gate != nullptr) {
                    const float2 gt = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(P.gate + k));
                    v.x = bf16r(v.x * gt.x);
                    v.y = bf16r(v.y * gt.y);
                }
                v.x = bf16r(h.x + v.x);
                v.y = bf16r(h.y + v.y);
                if (P.h_out != nullptr) {
                    *reinterpret_cast<__nv_bfloat162*>(P.h_out + static_cast<size_t>(m) * K + k) =
                        __floats2bfloat162_rn(v.x, v.y);
                }
            }
            row[k] = v.x;
            row[k + 1] = v.y;
        }
    }
    __syncthreads();

    // ---- normalise ---------------------------------------------------------------------------
    if (P.mode == TPB200_ROW_RMSNORM || P.mode == TPB200_ROW_ADARMS) {
        float ss = 0.0f;
        for (int k = tid; k < K; k += kThreads) ss += row[k] * row[k];
        ss = block_sum(ss, red);
        const float r = rsqrtf(ss / static_cast<float>(K) + P.eps);
        for (int k = tid; k < K; k += kThreads) {
            float v = row[k] * r;
            if (P.mode == TPB200_ROW_RMSNORM) {
                v = v * (1.0f + __bfloat162float(P.w0[k]));
            } else {
                v = v * (1.0f + __bfloat162float(P.w0[k])) + __bfloat162float(P.w1[k]);
            }
            row[k] = bf16r(v);
        }
    } else if (P.mode == TPB200_ROW_LAYERNORM) {
        float s = 0.0f;
        for (int k = tid; k < K; k += kThreads) s += row[k];
        const float mean = block_sum(s, red) / static_cast<float>(K);
        float ss = 0.0f;
        for (int k = tid; k < K; k += kThreads) {
            const float d = row[k] - mean;
            ss += d * d;
        }
        const float r = rsqrtf(block_sum(ss, red) / static_cast<float>(K) + P.eps);
        for (int k = tid; k < K; k += kThreads) {
            row[k] = bf16r((row[k] - mean) * r * __bfloat162float(P.w0[k]) + __bfloat162float(P.w1[k]));
        }
    }
    __syncthreads();

    if (P.y_out != nullptr) {
        for (int k = tid * 2; k < K; k += kThreads * 2) {
            *reinterpret_cast<__nv_bfloat162*>(P.y_out + static_cast<size_t>(m) * K + k) =
                __floats2bfloat162_rn(row[k], row[k + 1]);
        }
    }
    if (P.packed == nullptr) return;

    // ---- residual-piece quantisation (same arithmetic as nvfp4_quantize_pieces_kernel) --------
    float amax = 0.0f;
    for (int k = tid; k < K; k += kThreads) amax = fmaxf(amax, fabsf(row[k]));
    amax = block_max(amax, red);
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);
        e = 11 - ex;
    }
    const float pre = ldexpf(1.0f, e);
    if (tid == 0) P.row_scale[m] = ldexpf(1.0f, -e);
    const int nblk = K >> 4;
    for (int kb = tid; kb < P.kb_pad; kb += kThreads) {
        float r[16];
        const bool valid = kb < nblk;
        if (valid) {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = row[kb * 16 + i] * pre;
        }
        for (int p = 0; p < P.pieces; ++p) {
            uint8_t* sf_dst;
            uint8_t* code_dst;
            if (P.tiled) {
                // block (m / 128, kb / 16): [piece][128 rows][128 B, 16-byte chunks XOR-swizzled by row & 7],
                // then [piece][4 atoms of 512 B]
                const int rr = m & 127;
                const int j = kb & 15;
                uint8_t* blk = P.packed + (static_cast<size_t>(m >> 7) * (P.kb_pad >> 4) + (kb >> 4)) *
                                              (static_cast<size_t>(P.pieces) * 18432);
                code_dst = blk + p * 16384 + rr * 128 + ((((j >> 1) ^ (rr & 7))) << 4) + (j & 1) * 8;
                sf_dst = blk + P.pieces * 16384 + p * 2048 + (j >> 2) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (j & 3);
            } else {
                const int prow = p * P.piece_rows + m;
                sf_dst = P.sf + (static_cast<size_t>(prow >> 7) * (P.kb_pad >> 2) + (kb >> 2)) * 512 +
                         (prow & 31) * 16 + ((prow >> 5) & 3) * 4 + (kb & 3);
                code_dst = P.packed + static_cast<size_t>(prow) * P.pitch + kb * 8;
            }
            if (!valid) {
                *sf_dst = 0;
                continue;
            }
            uint32_t lo, hi;
            *sf_dst = quantize_block16_piece(r, lo, hi);
            *reinterpret_cast<uint2*>(code_dst) = make_uint2(lo, hi);
        }
    }
}

}  // namespace
}  // namespace tpb

extern "C" int tpb200_row_transform_quantize(const tpb200_rowop_args* a, tpb200_stream_t stream) {
    TPB_REQUIRE(a != nullptr && a->x != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(a->mode >= TPB200_ROW_NONE && a->mode <= TPB200_ROW_GELU_MUL, TPB200_ERR_ENUM);
    TPB_REQUIRE(a->M >= 1 && a->K >= 16 && a->K % 16 == 0 && a->K <= tpb::kMaxK, TPB200_ERR_SHAPE);
    TPB_REQUIRE(a->ldx >= (a->mode == TPB200_ROW_GELU_MUL ? 2 * a->K : a->K) && a->ldx % 2 == 0, TPB200_ERR_SHAPE);
    if (a->mode == TPB200_ROW_RMSNORM) TPB_REQUIRE(a->w0 != nullptr, TPB200_ERR_NULL);
    if (a->mode == TPB200_ROW_ADARMS || a->mode == TPB200_ROW_LAYERNORM) {
        TPB_REQUIRE(a->w0 != nullptr && a->w1 != nullptr, TPB200_ERR_NULL);
    }
    TPB_REQUIRE(a->packed != nullptr || a->y_out != nullptr || a->h_out != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(a->layout == TPB200_OPERANDS_ROWMAJOR || a->layout == TPB200_OPERANDS_TILED, TPB200_ERR_ENUM);
    if (a->packed != nullptr && a->layout == TPB200_OPERANDS_TILED) {
        TPB_REQUIRE(a->row_scale != nullptr, TPB200_ERR_NULL);
        TPB_REQUIRE(a->pieces >= 1 && a->pieces <= 3, TPB200_ERR_SHAPE);
        TPB_REQUIRE(tpb_aligned16(a->packed), TPB200_ERR_ALIGN);
    } else if (a->packed != nullptr) {
        TPB_REQUIRE(a->sf != nullptr && a->row_scale != nullptr, TPB200_ERR_NULL);
        TPB_REQUIRE(a->pieces >= 1 && a->pieces <= 4 && a->piece_rows >= a->M, TPB200_ERR_SHAPE);
        TPB_REQUIRE(a->pitch >= a->K / 2 && a->pitch % 16 == 0 && tpb_aligned16(a->packed) && tpb_aligned16(a->sf),
                    TPB200_ERR_ALIGN);
    }
    tpb::RowOpParams P;
    P.mode = a->mode;
    P.M = a->M;
    P.K = a->K;
    P.x = static_cast<const __nv_bfloat16*>(a->x);
    P.ldx = a->ldx;
    P.res_in = static_cast<const __nv_bfloat16*>(a->res_in);
    P.gate = static_cast<const __nv_bfloat16*>(a->gate);
    P.h_out = static_cast<__nv_bfloat16*>(a->h_out);
    P.w0 = static_cast<const __nv_bfloat16*>(a->w0);
    P.w1 = static_cast<const __nv_bfloat16*>(a->w1);
    P.eps = a->eps;
    P.y_out = static_cast<__nv_bfloat16*>(a->y_out);
    P.packed = static_cast<uint8_t*>(a->packed);
    P.pitch = a->pitch;
    P.sf = static_cast<uint8_t*>(a->sf);
    P.row_scale = a->row_scale;
    P.pieces = a->pieces;
    P.piece_rows = a->piece_rows;
    P.kb_pad = (a->K + 255) / 256 * 16;
    P.tiled = a->layout == TPB200_OPERANDS_TILED;
    const size_t smem = static_cast<size_t>(a->K) * sizeof(float);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(tpb::row_transform_quantize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 tpb::kMaxK * static_cast<int>(sizeof(float))) != cudaSuccess) {
            return TPB200_ERR_CUDA;
        }
    }
    tpb::row_transform_quantize_kernel<<<a->M, tpb::kThreads, smem, reinterpret_cast<cudaStream_t>(stream)>>>(P);
    return tpb_launch_status();
}
