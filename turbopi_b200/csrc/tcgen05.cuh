// Thin inline-PTX wrappers for the Blackwell tensor-core path: TMEM allocation,
// tcgen05.mma (block-scaled e2m1 x e2m1 with UE4M3 scales), tcgen05.cp (shared ->
// tensor memory for scale factors), tcgen05.ld, commit/fences, TMA tile loads, and the
// shared-memory / instruction descriptors they take.
#pragma once

#include <cuda.h>  // CUtensorMap (types only; the encode entry point is fetched at run time)

#include "common.cuh"

namespace tpb {
namespace tc {

// ------------------------------------------------------------------ tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols) {  // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void fence_before_thread_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_thread_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// all tcgen05 operations issued so far by this thread arrive on `bar` when they complete
__device__ __forceinline__ void commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor (sm_100 format):
//   [0,14)  start address >> 4      [16,30) leading-dim byte offset >> 4
//   [32,46) stride-dim byte offset >> 4   [46,48) version = 1   [61,64) swizzle mode
enum : uint64_t { kSwizzleNone = 0, kSwizzle128B = 2 };

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint64_t swizzle) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= swizzle << 61;
    return d;
}

// K-major operand tile stored as rows of 128 bytes under the 128-byte swizzle (what a TMA box of
// 128 bytes x R rows with CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
// `k_byte_offset` selects the 32-byte slice of one MMA inside the 128-byte row.
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t tile_smem_addr, uint32_t k_byte_offset) {
    return make_smem_desc(tile_smem_addr + k_byte_offset, 0, 1024, kSwizzle128B);
}

// Scale-factor atom for tcgen05.cp 32x128b: 32 rows of 16 bytes, contiguous, no swizzle
// (8-row core matrices 128 bytes apart, a single core matrix along K).
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t atom_smem_addr) {
    return make_smem_desc(atom_smem_addr, 0, 128, kSwizzleNone);
}

// The same descriptors split into 32-bit words.  The thread that issues the MMAs spends ~60 cycles per
// tcgen05 instruction when every descriptor is assembled with 64-bit arithmetic, and it is ONE thread: in
// a loop of 20-30 instructions per stage that is the kernel's critical path.  The upper word of a
// descriptor is a constant of its kind; the lower word is (shared-memory address >> 4) plus constants.
constexpr uint32_t kDescHiKmajorSw128 = (1024u >> 4) | (1u << 14) | (static_cast<uint32_t>(kSwizzle128B) << 29);
constexpr uint32_t kDescHiSfAtom = (128u >> 4) | (1u << 14);
__device__ __forceinline__ uint64_t desc_from_words(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// Instruction descriptor for kind::mxf4nvf4 (e2m1 x e2m1, UE4M3 scales per 16, K = 64), M = 128:
//   [7,10) A format = 1 (e2m1)  [10,13) B format = 1  [15],[16] K-major  [17,23) N >> 3
//   [23] scale format 0 = UE4M3  [24,29) M >> 4  [4,6)/[29,31) scale-factor byte ids = 0
__host__ __device__ constexpr uint32_t make_idesc_mxf4nvf4(int n) {
    return (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | ((128u >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]^T with block scales read from tensor memory
__device__ __forceinline__ void mma_mxf4nvf4(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t tmem_sfa, uint32_t tmem_sfb, uint32_t accumulate) {
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(tmem_sfa), "r"(tmem_sfb)
        : "memory");
}

// 32 rows x 16 bytes of shared memory -> tensor-memory lanes 0..31 (4 columns), replicated to the
// other three 32-lane quarters
__device__ __forceinline__ void cp_sf_32x128b(uint32_t tmem_dst, uint64_t sf_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_dst), "l"(sf_desc) : "memory");
}

// 32 consecutive fp32 columns of this thread's lane (warp w of a warpgroup reads lanes 32*(w%4)..)
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ------------------------------------------------------------------ TMA tile load (into this CTA only)
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], "
        "[%6];" ::"r"(smem_u32(smem_dst)),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        " .reg .pred p;\n"
        " elect.sync _|p, 0xffffffff;\n"
        " selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

}  // namespace tc

// ------------------------------------------------------------------ host: tensor maps
// 2-D byte tensor [rows, row_bytes] with pitch `pitch_bytes`, box 128 bytes x box_rows, 128-byte swizzle.
// Returns false if the driver entry point is unavailable or refuses the shape.
bool make_tensor_map_bytes_sw128(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                                 uint64_t pitch_bytes, uint32_t box_rows);

// bf16 tensor of 2..5 dimensions (dims[0] contiguous, strides_bytes[i] = byte stride of dims[i + 1], multiples of
// 16), box[0] <= 64 elements, 128-byte swizzle, zero fill past the end of every dimension.
bool make_tensor_map_bf16_nd_sw128(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                   const uint64_t* strides_bytes, const uint32_t* box);

}  // namespace tpb
