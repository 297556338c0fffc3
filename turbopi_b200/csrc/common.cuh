// Device-side helpers shared by the sm_100a kernels: mbarrier + bulk-copy (TMA)
// wrappers with bounded waits, programmatic-dependent-launch controls, 4-bit
// decoders and small numeric utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/turbopi_b200.h"

namespace tpb {

// ---------------------------------------------------------------------------
// Device error word.  A kernel whose bounded wait runs out records where it gave
// up here and returns; the host reads it with tpb200_device_error().
// ---------------------------------------------------------------------------
// The word is per translation unit (no relocatable device code needed); each kernel file
// exports a reader built from read_device_error() and tpb200_device_error() polls them all.
static __device__ int g_device_error = 0;

enum DeviceErrorCode : int {
    kErrNone = 0,
    kErrGemvFullBarrierTimeout = 101,
    kErrGemvEmptyBarrierTimeout = 102,
    kErrGemvUnitQueueTimeout = 103,
    kErrGemmTmaBarrierTimeout = 201,
    kErrGemmMmaBarrierTimeout = 202,
    kErrGemmEpilogueBarrierTimeout = 203,
    kErrGemmEmptyBarrierTimeout = 204,
    kErrGemmSplitTimeout = 205,
    kErrAttnBarrierTimeout = 301,
};

__device__ __forceinline__ void record_error(int code) { atomicCAS(&g_device_error, 0, code); }

// ---------------------------------------------------------------------------
// Shared-memory barriers and bulk async copies
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for a phase with a wall-clock bound (about a second at any SM clock).
// Returns false when the bound ran out; the caller records an error and leaves.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit_cycles = 2000000000LL) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (true) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
        }
        if (clock64() - start > limit_cycles) return false;
    }
}

// 1-D bulk copy global -> this CTA's shared memory, completion counted on `bar`.
// Both addresses 16-byte aligned, `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// The same copy with an L2 eviction hint: data that is read exactly once (a weight stream) should not push
// small, reused data (activations, scratch, the next kernel's inputs) out of L2.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
__device__ __forceinline__ void bulk_copy_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue (weight prefetch) while this one is still running, and
// wait for the previous kernel's results before touching dependent data.
// Both are no-ops when the launch did not opt in.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior_grids() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---------------------------------------------------------------------------
// 4-bit decoders.  A 32-bit word holds 8 codes, code i at bits 4i (byte j of a row
// holds k = 2j in its low nibble and k = 2j+1 in its high nibble).
// ---------------------------------------------------------------------------

// e2m1: h[p] = (value(k = 2p), value(k = 2p + 1)) as exact fp16.
__device__ __forceinline__ void decode_e2m1x8(uint32_t w, __half2 (&h)[4]) {
    uint32_t r0, r1, r2, r3;
    asm("{\n"
        " .reg .b8 b0, b1, b2, b3;\n"
        " mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n"
        " cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n"
        " cvt.rn.f16x2.e2m1x2 %3, b3;\n"
        "}\n"
        : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
        : "r"(w));
    h[0] = *reinterpret_cast<__half2*>(&r0);
    h[1] = *reinterpret_cast<__half2*>(&r1);
    h[2] = *reinterpret_cast<__half2*>(&r2);
    h[3] = *reinterpret_cast<__half2*>(&r3);
}

// unsigned int4 with zero point 8: h[p] = (q(k = p) - 8, q(k = p + 4) - 8), exact fp16.
// Note the pairing differs from e2m1: activations are packed to match (pack_x_*).
__device__ __forceinline__ void decode_u4x8_minus8(uint32_t w, __half2 (&h)[4]) {
    const uint32_t kMagic = 0x64006400u;              // 1024.0 in both halves
    const uint32_t k1032 = 0x64086408u;               // 1032.0
    const uint32_t kSixteenth = 0x2C002C00u;          // 1/16
    const uint32_t kMinus72 = 0xD480D480u;            // -72.0
    uint32_t lo0 = (w & 0x000F000Fu) | kMagic;        // 1024 + q0 | 1024 + q4
    uint32_t hi0 = (w & 0x00F000F0u) | kMagic;        // 1024 + 16 q1 | 1024 + 16 q5
    uint32_t w2 = w >> 8;
    uint32_t lo1 = (w2 & 0x000F000Fu) | kMagic;       // q2 | q6
    uint32_t hi1 = (w2 & 0x00F000F0u) | kMagic;       // q3 | q7
    h[0] = __hsub2(*reinterpret_cast<__half2*>(&lo0), *reinterpret_cast<const __half2*>(&k1032));
    h[1] = __hfma2(*reinterpret_cast<__half2*>(&hi0), *reinterpret_cast<const __half2*>(&kSixteenth),
                   *reinterpret_cast<const __half2*>(&kMinus72));
    h[2] = __hsub2(*reinterpret_cast<__half2*>(&lo1), *reinterpret_cast<const __half2*>(&k1032));
    h[3] = __hfma2(*reinterpret_cast<__half2*>(&hi1), *reinterpret_cast<const __half2*>(&kSixteenth),
                   *reinterpret_cast<const __half2*>(&kMinus72));
}

// two E4M3 bytes -> two floats (exact)
__device__ __forceinline__ float2 decode_e4m3x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return __half22float2(*reinterpret_cast<__half2*>(&r));
}

__device__ __forceinline__ float decode_e4m3(uint8_t v) { return decode_e4m3x2(static_cast<uint16_t>(v)).x; }

// float -> E4M3 byte, round-to-nearest-even, saturating to +-448
__device__ __forceinline__ uint8_t encode_e4m3(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return static_cast<uint8_t>(r & 0xFF);
}

// two floats -> one byte of e2m1 codes (lo in the low nibble), round-to-nearest-even, saturating at 6
__device__ __forceinline__ uint32_t encode_e2m1x2(float lo, float hi) {
    uint16_t r;
    asm("{\n"
        " .reg .b8 t;\n"
        " cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n"
        " cvt.u16.u8 %0, t;\n"
        "}\n"
        : "=h"(r)
        : "f"(hi), "f"(lo));
    return r;
}

// one byte of e2m1 codes -> (value of low nibble, value of high nibble)
__device__ __forceinline__ float2 decode_e2m1x2(uint32_t byte) {
    uint32_t r;
    const uint16_t b = static_cast<uint16_t>(byte);
    asm("{\n"
        " .reg .b8 lo, hi;\n"
        " mov.b16 {lo, hi}, %1;\n"
        " cvt.rn.f16x2.e2m1x2 %0, lo;\n"
        "}\n"
        : "=r"(r)
        : "h"(b));
    return __half22float2(*reinterpret_cast<__half2*>(&r));
}

// One residual piece of a 16-element block: chooses the UE4M3 scale (rounded up so nothing clips),
// returns the 16 codes in (lo, hi) and leaves in r what the piece could not represent.
__device__ __forceinline__ uint8_t quantize_block16_piece(float (&r)[16], uint32_t& lo, uint32_t& hi) {
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) bmax = fmaxf(bmax, fabsf(r[i]));
    const float want = bmax * (1.0f / 6.0f);
    uint8_t code = encode_e4m3(want);
    float s = decode_e4m3(code);
    if (s < want && code < 0x7E) {   // next representable scale up (positive codes are monotonic)
        code += 1;
        s = decode_e4m3(code);
    }
    const float inv = s > 0.0f ? 1.0f / s : 0.0f;
    lo = 0;
    hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t byte = encode_e2m1x2(r[2 * i] * inv, r[2 * i + 1] * inv);
        const float2 q = decode_e2m1x2(byte);
        r[2 * i] = fmaf(-q.x, s, r[2 * i]);
        r[2 * i + 1] = fmaf(-q.y, s, r[2 * i + 1]);
        if (i < 4) lo |= byte << (8 * i);
        else hi |= byte << (8 * (i - 4));
    }
    return code;
}

// The same piece for a 16-element block held by TWO adjacent lanes (eight elements each, the even lane the
// first eight): the block maximum crosses the pair with one shuffle, both lanes derive the same scale, each
// returns the 32-bit word of its own eight codes.  Bit-identical to quantize_block16_piece.  All 32 lanes of
// the warp must call it together.
__device__ __forceinline__ uint8_t quantize_half8_piece(float (&r)[8], uint32_t& word) {
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) bmax = fmaxf(bmax, fabsf(r[i]));
    bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 1));
    const float want = bmax * (1.0f / 6.0f);
    uint8_t code = encode_e4m3(want);
    float s = decode_e4m3(code);
    if (s < want && code < 0x7E) {
        code += 1;
        s = decode_e4m3(code);
    }
    const float inv = s > 0.0f ? 1.0f / s : 0.0f;
    word = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t byte = encode_e2m1x2(r[2 * i] * inv, r[2 * i + 1] * inv);
        const float2 q = decode_e2m1x2(byte);
        r[2 * i] = fmaf(-q.x, s, r[2 * i]);
        r[2 * i + 1] = fmaf(-q.y, s, r[2 * i + 1]);
        word |= byte << (8 * i);
    }
    return code;
}

// Exponent e of the row pre-scale 2^e that brings a row's largest magnitude into [1024, 2048)
__device__ __forceinline__ int prescale_exponent(float amax) {
    int e = 0;
    if (amax > 0.0f && amax < 3.0e38f) {
        int ex;
        frexpf(amax, &ex);
        e = 11 - ex;
    }
    return e;
}

// ---------------------------------------------------------------------------
// Scalars of a run-time dtype
// ---------------------------------------------------------------------------
__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
    if (dtype == TPB200_F32) return static_cast<const float*>(p)[i];
    if (dtype == TPB200_F16) return __half2float(static_cast<const __half*>(p)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__device__ __forceinline__ void store_from_float(void* p, int dtype, size_t i, float v) {
    if (dtype == TPB200_F32) {
        static_cast<float*>(p)[i] = v;
    } else if (dtype == TPB200_F16) {
        static_cast<__half*>(p)[i] = __float2half_rn(v);
    } else {
        static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
    }
}

// 16 consecutive elements (16-element aligned) of a run-time dtype as floats, with 128-bit loads
__device__ __forceinline__ void load16_as_float(const void* p, int dtype, size_t e0, float (&v)[16]) {
    if (dtype == TPB200_F32) {
        const float4* q = reinterpret_cast<const float4*>(static_cast<const float*>(p) + e0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 f = __ldg(q + i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
    } else {
        const uint4* q = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p) + e0);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 u = __ldg(q + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = dtype == TPB200_F16
                                     ? __half22float2(*reinterpret_cast<const __half2*>(&w[j]))
                                     : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[j]));
                v[8 * i + 2 * j] = f.x;
                v[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
}

__device__ __forceinline__ float gelu_tanh(float x) {
    const float kSqrt2OverPi = 0.7978845608028654f;
    float inner = kSqrt2OverPi * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(inner));
}

__device__ __forceinline__ float silu(float x) { return x / (1.0f + expf(-x)); }

__device__ __forceinline__ float apply_activation(float v, int act) {
    if (act == TPB200_ACT_GELU) return gelu_tanh(v);
    if (act == TPB200_ACT_SILU) return silu(v);
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace tpb

static inline int read_device_error(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, tpb::g_device_error, sizeof(int)) != cudaSuccess) return TPB200_ERR_CUDA;
    if (clear && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(tpb::g_device_error, &zero, sizeof(int));
    }
    return v;
}

// ---------------------------------------------------------------------------
// Host-side argument checks shared by the entry points
// ---------------------------------------------------------------------------
#define TPB_REQUIRE(cond, code) \
    do {                        \
        if (!(cond)) return (code); \
    } while (0)

static inline bool tpb_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline bool tpb_valid_dtype(int d) { return d == TPB200_F32 || d == TPB200_F16 || d == TPB200_BF16; }
static inline int tpb_dtype_size(int d) { return d == TPB200_F32 ? 4 : 2; }
static inline int tpb_launch_status() { return cudaGetLastError() == cudaSuccess ? TPB200_OK : TPB200_ERR_CUDA; }
