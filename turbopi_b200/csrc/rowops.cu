// Row-wise glue fused with the activation quantiser of the tensor-core GEMM.
//
// Between two linears the model only does row-local work (residual add, RMSNorm / adaptive
// RMSNorm / LayerNorm, GELU(gate) * up).  Each of these is one kernel here that reads the bf16
// inputs once, does the arithmetic in fp32 with the roundings the PyTorch modules apply
// (openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:49-129,
// 212-230), and writes the result straight in the GEMM's operand format: residual e2m1 pieces +
// UE4M3 block scales + the per-row power-of-two multiplier (see nvfp4_gemm.cu).  A bf16 copy of
// the transformed row and the updated residual stream are written only when asked for.
// One CTA per row; every thread keeps its 16-element blocks in registers (K <= 16384).
#include <algorithm>

#include "common.cuh"

namespace tpb {
namespace {

constexpr int kThreads = 512;    // up to two 16-element blocks per thread: K <= 16384
constexpr int kMaxK = 16384;

struct RowOpParams {
    int mode;
    int M, K;
    const __nv_bfloat16* x;        // main input [M, ldx] (GELU_MUL / SILU_MUL: [M, 2K] = gate | up)
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

// Block-wide reductions for any multiple of 32 threads up to 256.
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t += red[i];
    return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) t = fmaxf(t, red[i]);
    return t;
}

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// GELU (tanh form) as x * sigmoid(2 z), z = sqrt(2/pi) (x + 0.044715 x^3): the same function as
// 0.5 x (1 + tanh z) without the cancellation in 1 + tanh z for negative x, so the hardware exp and
// divide keep ~1e-6 relative accuracy everywhere.
__device__ __forceinline__ float gelu_tanh_hw(float x) {
    const float z2 = 1.5957691216057308f * (x + 0.044715f * x * x * x);
    return __fdividef(x, 1.0f + __expf(-z2));
}

// E = 8 or 16 consecutive bf16 (16-byte aligned) <-> floats
template <int E>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float (&v)[E]) {
    const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
    for (int i = 0; i < E / 8; ++i) {
        const uint4 u = __ldg(q + i);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
            v[8 * i + 2 * j] = f.x;
            v[8 * i + 2 * j + 1] = f.y;
        }
    }
}

template <int E>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const float (&v)[E]) {
    uint32_t w[E / 2];
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
        __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&b);
    }
    uint4* q = reinterpret_cast<uint4*>(p);
#pragma unroll
    for (int i = 0; i < E / 8; ++i) q[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
}

// One CTA per row; thread t owns the 16-element blocks t and (for rows longer than 8192) t + T and keeps
// them in registers from the global load to the code store; the only shared memory is the scratch of the
// block-wide reductions.  512 threads x 2 blocks instead of 1024 x 1 for the longest rows: two CTAs fit an
// SM's register file, so one row's reductions overlap the other's arithmetic.
template <int NB, int E>
__global__ void __launch_bounds__(kThreads) row_transform_quantize_kernel(const __grid_constant__ RowOpParams P) {
    __shared__ float red[kThreads / 32];
    // under programmatic dependent launch this kernel may start while its producer still runs
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int m = blockIdx.x;
    const int K = P.K;
    const int T = blockDim.x;
    const int tid = threadIdx.x;
    const int nblk = K >> 4;
    const int nunit = K / E;                    // units of E elements: whole 16-element blocks (E = 16) or halves (E = 8)
    float v[NB][E];

    // ---- load (+ residual) ------------------------------------------------------------------
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        const int u = tid + j * T;
        if (u >= nunit) {
#pragma unroll
            for (int i = 0; i < E; ++i) v[j][i] = 0.0f;
            continue;
        }
        const int k = u * E;
        if (P.mode == TPB200_ROW_GELU_MUL || P.mode == TPB200_ROW_SILU_MUL) {
            float g[E], up[E];
            load_bf16<E>(P.x + static_cast<size_t>(m) * P.ldx + k, g);
            load_bf16<E>(P.x + static_cast<size_t>(m) * P.ldx + K + k, up);
            if (P.mode == TPB200_ROW_GELU_MUL) {
#pragma unroll
                for (int i = 0; i < E; ++i) v[j][i] = bf16r(bf16r(gelu_tanh_hw(g[i])) * up[i]);
            } else {
#pragma unroll
                for (int i = 0; i < E; ++i) v[j][i] = bf16r(bf16r(__fdividef(g[i], 1.0f + __expf(-g[i]))) * up[i]);
            }
        } else {
            load_bf16<E>(P.x + static_cast<size_t>(m) * P.ldx + k, v[j]);
            if (P.res_in != nullptr) {
                float h[E];
                load_bf16<E>(P.res_in + static_cast<size_t>(m) * K + k, h);
                if (P.gate != nullptr) {
                    float gt[E];
                    load_bf16<E>(P.gate + k, gt);
#pragma unroll
                    for (int i = 0; i < E; ++i) v[j][i] = bf16r(v[j][i] * gt[i]);
                }
#pragma unroll
                for (int i = 0; i < E; ++i) v[j][i] = bf16r(h[i] + v[j][i]);
                if (P.h_out != nullptr) store_bf16<E>(P.h_out + static_cast<size_t>(m) * K + k, v[j]);
            }
        }
    }

    // ---- normalise ---------------------------------------------------------------------------
    if (P.mode == TPB200_ROW_RMSNORM || P.mode == TPB200_ROW_ADARMS) {
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int i = 0; i < E; ++i) ss += v[j][i] * v[j][i];
        }
        ss = block_sum(ss, red);
        const float r = rsqrtf(ss / static_cast<float>(K) + P.eps);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int u = tid + j * T;
            if (u >= nunit) continue;
            float w0[E];
            load_bf16<E>(P.w0 + u * E, w0);
            if (P.mode == TPB200_ROW_RMSNORM) {
#pragma unroll
                for (int i = 0; i < E; ++i) v[j][i] = bf16r(v[j][i] * r * (1.0f + w0[i]));
            } else {
                float w1[E];
                load_bf16<E>(P.w1 + u * E, w1);
#pragma unroll
                for (int i = 0; i < E; ++i) v[j][i] = bf16r(v[j][i] * r * (1.0f + w0[i]) + w1[i]);
            }
        }
    } else if (P.mode == TPB200_ROW_LAYERNORM) {
        float sm = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
#pragma unroll
            for (int i = 0; i < E; ++i) sm += v[j][i];
        }
        const float mean = block_sum(sm, red) / static_cast<float>(K);
        float ss = 0.0f;
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            if (tid + j * T >= nunit) continue;
#pragma unroll
            for (int i = 0; i < E; ++i) {
                const float d = v[j][i] - mean;
                ss += d * d;
            }
        }
        const float r = rsqrtf(block_sum(ss, red) / static_cast<float>(K) + P.eps);
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int u = tid + j * T;
            if (u >= nunit) continue;
            float w0[E], w1[E];
            load_bf16<E>(P.w0 + u * E, w0);
            load_bf16<E>(P.w1 + u * E, w1);
#pragma unroll
            for (int i = 0; i < E; ++i) v[j][i] = bf16r((v[j][i] - mean) * r * w0[i] + w1[i]);
        }
    }

    if (P.y_out != nullptr) {
#pragma unroll
        for (int j = 0; j < NB; ++j) {
            const int u = tid + j * T;
            if (u < nunit) store_bf16<E>(P.y_out + static_cast<size_t>(m) * K + u * E, v[j]);
        }
    }
    if (P.packed == nullptr) return;

    // ---- residual-piece quantisation (same arithmetic as nvfp4_quantize_pieces_kernel) --------
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < NB; ++j) {
#pragma unroll
        for (int i = 0; i < E; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
    }
    amax = block_max(amax, red);
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);
        e = 11 - ex;
    }
    const float pre = ldexpf(1.0f, e);
    if (tid == 0) P.row_scale[m] = ldexpf(1.0f, -e);
#pragma unroll
    for (int j = 0; j < NB; ++j) {
        // E = 16: this thread's whole block kb.  E = 8: half hb of block kb; the two lanes of a block derive the
        // same scale (one shuffle for the block maximum), so every thread of the warp takes part (the launch has
        // 2 * kb_pad threads, a multiple of 32: no thread is past the padded row)
        const int u = tid + j * T;
        const int kb = E == 16 ? u : u >> 1;
        const int hb = E == 16 ? 0 : u & 1;
        if (E == 16 && kb >= P.kb_pad) continue;
        const bool valid = kb < nblk;
#pragma unroll
        for (int i = 0; i < E; ++i) v[j][i] = valid ? v[j][i] * pre : 0.0f;
        for (int p = 0; p < P.pieces; ++p) {
            uint8_t* sf_dst;
            uint8_t* code_dst;
            if (P.tiled) {
                // block (m / 128, kb / 16): [piece][128 rows][128 B, 16-byte chunks XOR-swizzled by row & 7],
                // then [piece][4 atoms of 512 B]
                const int rr = m & 127;
                const int jj = kb & 15;
                uint8_t* blk = P.packed + (static_cast<size_t>(m >> 7) * (P.kb_pad >> 4) + (kb >> 4)) *
                                              (static_cast<size_t>(P.pieces) * 18432);
                code_dst = blk + p * 16384 + rr * 128 + ((((jj >> 1) ^ (rr & 7))) << 4) + (jj & 1) * 8;
                sf_dst = blk + P.pieces * 16384 + p * 2048 + (jj >> 2) * 512 + (rr & 31) * 16 + (rr >> 5) * 4 + (jj & 3);
            } else {
                const int prow = p * P.piece_rows + m;
                sf_dst = P.sf + (static_cast<size_t>(prow >> 7) * (P.kb_pad >> 2) + (kb >> 2)) * 512 +
                         (prow & 31) * 16 + ((prow >> 5) & 3) * 4 + (kb & 3);
                code_dst = P.packed + static_cast<size_t>(prow) * P.pitch + kb * 8;
            }
            if constexpr (E == 16) {
                if (!valid) {
                    *sf_dst = 0;
                    continue;
                }
                uint32_t lo, hi;
                *sf_dst = quantize_block16_piece(v[j], lo, hi);
                *reinterpret_cast<uint2*>(code_dst) = make_uint2(lo, hi);
            } else {
                uint32_t word;
                const uint8_t code = quantize_half8_piece(v[j], word);   // zeros in: zero scale, zero codes
                if (hb == 0) *sf_dst = code;
                if (valid) *reinterpret_cast<uint32_t*>(code_dst + hb * 4) = word;
            }
        }
    }
}

}  // namespace
}  // namespace tpb

extern "C" int tpb200_row_transform_quantize(const tpb200_rowop_args* a, tpb200_stream_t stream) {
    TPB_REQUIRE(a != nullptr && a->x != nullptr, TPB200_ERR_NULL);
    TPB_REQUIRE(a->mode >= TPB200_ROW_NONE && a->mode <= TPB200_ROW_SILU_MUL, TPB200_ERR_ENUM);
    TPB_REQUIRE(a->M >= 1 && a->K >= 16 && a->K % 16 == 0 && a->K <= tpb::kMaxK, TPB200_ERR_SHAPE);
    TPB_REQUIRE(a->ldx >= (a->mode >= TPB200_ROW_GELU_MUL ? 2 * a->K : a->K) && a->ldx % 8 == 0, TPB200_ERR_SHAPE);
    TPB_REQUIRE(tpb_aligned16(a->x) && tpb_aligned16(a->res_in) && tpb_aligned16(a->gate) && tpb_aligned16(a->h_out) &&
                    tpb_aligned16(a->w0) && tpb_aligned16(a->w1) && tpb_aligned16(a->y_out),
                TPB200_ERR_ALIGN);
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
    // rows of up to 4096 elements: two threads per 16-element block (the three residual pieces are a dependent
    // chain per block; halving it is what a latency-bound launch gains from); longer rows: one or two blocks per thread
    const bool halves = a->packed != nullptr && P.kb_pad <= tpb::kThreads / 2;
    const int threads = halves ? 2 * P.kb_pad : std::min(tpb::kThreads, (P.kb_pad + 31) / 32 * 32);
    TPB_REQUIRE((a->flags & ~TPB200_FLAG_PDL) == 0, TPB200_ERR_ENUM);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a->M, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    if (a->flags & TPB200_FLAG_PDL) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    const cudaError_t err = halves ? cudaLaunchKernelEx(&cfg, tpb::row_transform_quantize_kernel<1, 8>, P)
                            : P.kb_pad <= tpb::kThreads
                                ? cudaLaunchKernelEx(&cfg, tpb::row_transform_quantize_kernel<1, 16>, P)
                                : cudaLaunchKernelEx(&cfg, tpb::row_transform_quantize_kernel<2, 16>, P);
    if (err != cudaSuccess) return TPB200_ERR_CUDA;
    return tpb_launch_status();
}
