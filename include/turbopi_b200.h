/*
 * turbopi_b200 -- C ABI of the B200 (sm_100a) kernels behind TurboPi's quantized
 * Pi0.5 inference plugins.
 *
 * Conventions for every entry point:
 *   - all tensor pointers are caller-owned DEVICE memory, row-major, 16-byte aligned;
 *   - the call only enqueues work on `stream` (no allocation, no synchronisation,
 *     no global mutable state), so it may be captured in a CUDA graph and is safe
 *     to call concurrently on different streams -- except tpb200_nvfp4_gemv_tc_static,
 *     whose scratch is one array shared by every call on a device (see there); launches that may
 *     overlap must not share a workspace;
 *   - the device is the calling thread's current device;
 *   - `tpb200_*` functions return TPB200_OK or a negative tpb200_status; arguments
 *     are validated on the host before anything is launched;
 *   - functions that carry the reference's own names and signatures return void
 *     as theirs do and report a bad argument through tpb200_last_error().
 *
 * File/line citations name the reference interface each entry point replaces
 * (paths inside the TurboPi repository).
 */
#ifndef TURBOPI_B200_H_
#define TURBOPI_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* tpb200_stream_t; /* == cudaStream_t */

typedef enum {
    TPB200_OK = 0,
    TPB200_ERR_NULL = -1,      /* a required pointer is NULL */
    TPB200_ERR_SHAPE = -2,     /* a dimension is out of the supported range */
    TPB200_ERR_ALIGN = -3,     /* a pointer or row pitch is not 16-byte aligned */
    TPB200_ERR_ENUM = -4,      /* unknown dtype / layout / activation / flag */
    TPB200_ERR_CUDA = -5,      /* the CUDA runtime refused the launch */
    TPB200_ERR_WORKSPACE = -6, /* workspace missing or too small */
    TPB200_ERR_DEVICE = -7     /* a kernel gave up on a bounded wait (tpb200_device_error) */
} tpb200_status;

/* element types; values match the reference's DataType enum
 * (openpi/nvfp4_packed_plugin/src/nvfp4_packed_kernel.cu:411-415) */
enum { TPB200_F32 = 0, TPB200_F16 = 1, TPB200_BF16 = 2 };

/* fused activations; values match the reference's ActivationType
 * (openpi/nvfp4_packed_plugin/src/nvfp4_packed_plugin.h:44-48) */
/* TPB200_ACT_GEGLU (tensor-core GEMM with tiled operands only): B stacks a gate and an up projection,
 * every 256-row block = 128 gate rows followed by the 128 matching up rows; the output has N / 2
 * columns, out[m, j] = bf16(gelu_tanh(bf16(gate_j))) * bf16(up_j)  (GemmaMLP,
 * openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:212-230). */
enum { TPB200_ACT_NONE = 0, TPB200_ACT_GELU = 1, TPB200_ACT_SILU = 2, TPB200_ACT_GEGLU = 3 };

/* block-scale encodings */
enum { TPB200_SCALE_F32 = 0, TPB200_SCALE_E4M3 = 1, TPB200_SCALE_F16 = 2, TPB200_SCALE_BF16 = 3 };

/* INT4 weight layouts */
enum {
    TPB200_INT4_KBLOCK = 0,  /* (K/32, N, 4) int32 + (K/32, N) fp16 scales: W4A16Packer's order,
                                openpi/src/openpi/utils/w4a16_packer.py:129-174 */
    TPB200_INT4_ROWMAJOR = 1, /* (N, K/8) int32 + (N, K/group) scales, 8 codes per word along K */
    TPB200_INT4_PLUGIN = 2    /* signed nibbles [N, K/2] bytes + bf16 scale / optional zero per 128: the w4a16 plugin's format */
};

/* launch flags */
enum {
    TPB200_FLAG_NONE = 0,
    TPB200_FLAG_PDL = 1 /* launch with programmatic stream serialisation: the kernel prefetches its
                           weights while the previous kernel in the stream is still running, and
                           waits for that kernel before it reads activations or writes outputs.
                           Requirement on the caller: weight images, scales and bias must be COMPLETE
                           before a launch with this flag is enqueued -- a kernel that prepares them
                           (tpb200_nvfp4_tile_weights, quantizeWeightToNVFP4, ...) must not be the
                           launch's immediate predecessor in the stream; put a stream or event
                           synchronisation, or any launch without the flag, in between. */
};

int tpb200_version(void);
const char* tpb200_status_string(int status);
/* last non-OK status produced on this host thread by a void-returning entry point (and clears it) */
int tpb200_last_error(void);
/* code recorded by a kernel whose bounded wait ran out on the current device, 0 if none; synchronises
 * the device.  `clear` != 0 resets the word.
 * Recovery: a kernel that gave up may have left its split-K counters non-zero.  After a non-zero code
 * every workspace that was passed to a GEMM / GEMV / attention launch since the last check must be set
 * to zero again (cudaMemsetAsync) before it is reused; results of the failed launch are undefined. */
int tpb200_device_error(int clear);

/* ---------------------------------------------------------------------------------------------
 * W4A16 INT4 GEMV/GEMM for decode shapes (M <= 16).
 *   out[m, n] = sum_k x[m, k] * (q[n, k] - 8) * scale[n, k / group] (+ bias[n])
 * q are unsigned 4-bit codes (zero point 8), code i of a word at bits 4i.
 * Replaces torch.ops.openpi.w4a16_gemv / the TVM gemv_vec128 kernel
 * (openpi/src/openpi/ops/w4a16_gemv.py:56-102,244-294) for layout KBLOCK, group 32, fp16
 * activations, fp32 output, M == 1; ROWMAJOR with group 128 is the benchmark layout.
 * scales are fp16 (TPB200_SCALE_F16) or bf16.  fp32 accumulation.
 * ------------------------------------------------------------------------------------------- */
int tpb200_w4a16_gemv(const void* x, int x_dtype, const void* weight_packed, const void* scales,
                      int scale_dtype, const void* bias, int bias_dtype, void* out, int out_dtype, int M,
                      int N, int K, int group_size, int layout, int flags, tpb200_stream_t stream);

/* W4A16 GEMM for more than 16 tokens on the tensor cores: INT4 weights are dequantised to bf16 on their way
 * into shared memory (once per CTA and K stage, shared by up to 384 token rows) and multiplied by tcgen05.mma
 * kind::f16; fp32 accumulation.  out = alpha * x @ dequant(W)^T + bias + beta * out.
 *   layout TPB200_INT4_PLUGIN: w = q * scale + zero, the operands of w4a16GemmForward
 *          (openpi/w4a16_plugin/src/w4a16_gemm_kernel.cu:54-153,336-406 is the reference's mixed-input GEMM);
 *   layout TPB200_INT4_KBLOCK: W4A16Linear's buffers, w = (q - 8) * scale (fp16, per 32; `zeros` must be NULL),
 *          replacing its dequantise + F.linear branch (openpi/src/openpi/modules/w4a16_linear.py:256-268).
 * x bf16 [M, K] contiguous, K % 128 == 0, N % 8 == 0, ldo = row stride of out in elements (0 = N). */
int tpb200_w4a16_gemm(const void* x, const void* weight, const void* scales, const void* zeros, const void* bias,
                      int bias_dtype, void* out, int out_dtype, int M, int N, int K, int ldo, int layout, float alpha,
                      float beta, int flags, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * NVFP4 weight-only GEMV/GEMM for decode shapes (M <= 16).
 *   out[m, n] = act(global_scale * sum_k x[m,k] * xs[m,k/block] * E2M1[code[n,k]] * ws[n,k/block] + bias[n])
 * weight_packed [N, K/2] bytes (even k in the low nibble), weight_scales [N, K/block] fp32 or E4M3,
 * block in {16, 32}; x_scales optional ([M, K/block], dtype of x).
 * Replaces nvfp4_gemv_v6 / nvfp4_gemv_w4a16 / nvfp4_gemv
 * (openpi/nvfp4_packed_plugin/src/nvfp4_gemv_v5.cu:430-476,
 *  openpi/nvfp4_packed_plugin/src/nvfp4_packed_torch.cu:173-290).
 * ------------------------------------------------------------------------------------------- */
int tpb200_nvfp4_gemv(const void* x, int x_dtype, const void* x_scales, const void* weight_packed,
                      const void* weight_scales, int scale_dtype, int block_size, float global_scale,
                      const void* bias, int bias_dtype, void* out, int out_dtype, int M, int N, int K,
                      int activation, int flags, tpb200_stream_t stream);

/* One launch over several independent NVFP4 GEMVs that share M, dtypes, block format and activation
 * (q/k/v, gate/up, or a whole stack of layers in a benchmark).  `count` <= TPB200_MAX_GROUP. */
#define TPB200_MAX_GROUP 64
typedef struct {
    const void* x;             /* [M, K] */
    const void* weight_packed; /* [N, K/2] */
    const void* weight_scales; /* [N, K/block] */
    const void* bias;          /* [N] or NULL */
    void* out;                 /* [M, N] */
    int N;
    int K;
    float global_scale;
    int out_stride;            /* elements between output rows; 0 = N */
} tpb200_gemv_problem;

int tpb200_nvfp4_gemv_grouped(const tpb200_gemv_problem* problems, int count, int x_dtype, int scale_dtype,
                              int block_size, int bias_dtype, int out_dtype, int M, int activation,
                              int flags, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * NVFP4 x NVFP4 block-scaled GEMM on tcgen05 tensor cores (prefix shapes, any M):
 *   out[M, N] = act(alpha * sum_k (a[m,k] sfa[m,k/16]) * (b[n,k] sfb[n,k/16]) + bias[n])
 * a_packed [M, a_pitch] / b_packed [N, b_pitch] bytes: e2m1 codes two per byte (even k low), pitches
 * multiples of 16 bytes; a_sf / b_sf: UE4M3 scales per 16 along K in 512-byte atoms of 128 rows x
 * 4 K-blocks (byte (r%32)*16 + (r/32)*4 + kb inside an atom), atoms ordered [row tile][K atom] with
 * K padded to a multiple of 256 -- tpb200_nvfp4_sf_bytes() gives the buffer size, padding scales
 * must be 0.  N % 8 == 0, K % 16 == 0.  bf16 or fp32 output with leading dimension ldo.
 * Replaces nvfp4_gemm.gemm / gemm_prepared / reorder_scales
 * (openpi/src/openpi/models_pytorch/nvfp4_extension/nvfp4_gemm.cu:216-304,330-429,451-549).
 * tpb200_nvfp4_quantize_act produces the A operand from bf16/fp16/fp32 activations with the
 * reference's per-block recipe (openpi/src/openpi/models_pytorch/nvfp4_mlp.py:88-173,606-608).
 * ------------------------------------------------------------------------------------------- */
size_t tpb200_nvfp4_sf_bytes(int rows, int K);
int tpb200_nvfp4_quantize_act(const void* x, int x_dtype, int ldx, void* packed, int packed_pitch,
                              void* sf_swizzled, int M, int K, tpb200_stream_t stream);
int tpb200_nvfp4_gemm(const void* a_packed, int a_pitch, const void* a_sf, const void* b_packed, int b_pitch,
                      const void* b_sf, float alpha, const void* bias_f32, int activation, void* out,
                      int out_dtype, int ldo, int M, int N, int K, int flags, tpb200_stream_t stream);

/* Extended form.  Adds (a) weight-only semantics on the tensor-core path: the A operand may be given as
 * `a_pieces` residual pieces of a bf16 activation matrix (tpb200_nvfp4_quantize_act_pieces: piece p of row
 * m at packed row p * a_piece_rows + m, a_piece_rows a multiple of 128, per-row power-of-two pre-scale
 * undone through a_row_scale), which the kernel sums in its accumulator; and (b) the fused QKV epilogue
 * that replaces fused_qkv_fp4 for prefix shapes (openpi/kv_fuse_plugin/src/fused_qkv_fp4.cu:382-467 plus
 * the RoPE + cache fill of openpi/src/openpi/models_pytorch/pi0_pytorch.py:455-473): B = [Wq; Wk; Wv]
 * with head_dim 256 and one KV head, rows tile-permuted (tile 2*head+half = head rows [64*half, 64*half+64)
 * then the same +128), rotary embedding applied to Q and K in bf16, Q written to qkv_q_out, K (post-RoPE)
 * and V rows written to qkv_k_rows / qkv_v_rows + m * 256 (pointers to the cache row of the first token). */
typedef struct {
    const void* a_packed; int a_pitch; const void* a_sf;
    int a_pieces; int a_piece_rows; const float* a_row_scale;
    const void* b_packed; int b_pitch; const void* b_sf;
    float alpha; const float* bias; int activation;
    void* out; int out_dtype; int ldo;
    int M, N, K;
    void* qkv_q_out; int qkv_ldq; int qkv_q_dim;
    void* qkv_k_rows; void* qkv_v_rows;
    const int* qkv_positions; const void* qkv_rope_cos; const void* qkv_rope_sin; /* bf16 [positions, 128] */
    /* Optional split-K scratch.  Shapes with fewer 128 x 128 output tiles than SMs split their K range over
     * several CTAs per tile when a workspace of at least tpb200_nvfp4_gemm_workspace_size() bytes is given
     * (a smaller one limits the split; NULL = never split).  Zero it ONCE after allocation: the kernel
     * leaves its counters at zero.  Launches that share a workspace must not overlap.  The partial sums
     * are added in a fixed order, so results do not depend on timing.
     * In a split launch the CTAs of a tile wait (bounded, ~1 s) for each other; the launch is a cooperative
     * launch, which the GPU places only when the whole grid fits, so launches on other streams cannot keep
     * partners out.  Each of two launches that may overlap needs a workspace of its own. */
    void* workspace; size_t workspace_bytes;
    /* Operand format.  TPB200_OPERANDS_ROWMAJOR (0): as described above.  TPB200_OPERANDS_TILED: a_packed and
     * b_packed point at pre-tiled images that carry their scales (a_sf, b_sf, pitches and a_piece_rows are
     * ignored), which the kernel streams in large contiguous requests into 128 x 256 output tiles -- the
     * fast path.  B image (tpb200_nvfp4_tile_weights makes it from the row-major operand, once per weight):
     * blocks [ceil(N/256)][ceil(K/256)] of 36864 bytes = 256 rows x 128 B of codes, 16-byte chunk c of row r
     * at chunk c ^ (r & 7), then the 2048-byte scale slabs (4 atoms) of rows 0..127 and 128..255.  A image
     * (tpb200_row_transform_quantize with TPB200_OPERANDS_TILED writes it): blocks [ceil(M/128)][ceil(K/256)]
     * of a_pieces * 18432 bytes = one 128-row code tile per piece in the same chunk pattern, then one scale
     * slab per piece; a_pieces <= 3.  Padding rows / K must hold zero scales. */
    int layout;
    /* TPB200_FLAG_PDL: launch with programmatic stream serialisation.  The kernel sets itself up (barriers,
     * tensor memory) while the previous kernel of the stream is still running and waits for it before it
     * reads an operand or writes a result. */
    int flags;
} tpb200_nvfp4_gemm_args;
enum { TPB200_OPERANDS_ROWMAJOR = 0, TPB200_OPERANDS_TILED = 1 };
size_t tpb200_nvfp4_gemm_workspace_size(int M, int N, int K, int a_pieces, int layout);
size_t tpb200_nvfp4_tiled_a_bytes(int M, int K, int pieces);
size_t tpb200_nvfp4_tiled_b_bytes(int N, int K);

/* Measurement utility (no counterpart in the reference): one CTA per SM issues `mmas_per_cta` block-scaled e2m1
 * MMAs of 128 x 256 x 64 (4,194,304 flops each) back to back on operands resident in shared memory -- no loads, no
 * epilogue.  Time the launch with events: SMs * mmas_per_cta * 4194304 / time is this GPU's FP4 tensor rate at the
 * clocks it runs at, the denominator the GEMM's rates are quoted against next to the nominal figure. */
int tpb200_measure_fp4_mma_rate(int mmas_per_cta, tpb200_stream_t stream);
int tpb200_nvfp4_tile_weights(const void* b_packed, int b_pitch, const void* b_sf, void* image, int N, int K,
                              tpb200_stream_t stream);
int tpb200_nvfp4_gemm_ex(const tpb200_nvfp4_gemm_args* args, tpb200_stream_t stream);
int tpb200_nvfp4_quantize_act_pieces(const void* x, int x_dtype, int ldx, void* packed, int packed_pitch,
                                     void* sf_swizzled, float* row_scale, int M, int K, int pieces,
                                     int piece_rows, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * NVFP4 weight-only GEMV for decode shapes (M <= 16) on the tensor cores: same result as
 * tpb200_nvfp4_gemv (E4M3 block-16 scales + global scale), no per-weight work on the SM.
 * w_image is the tensor-core GEMM's tiled B image (tpb200_nvfp4_tile_weights; blocks
 * [ceil(N/256)][ceil(K/256)] of 36864 bytes), so one copy of a weight serves prefill and decode.
 * Activations are first turned into `pieces` residual e2m1 operands by tpb200_nvfp4_quantize_act_tc:
 * x_image = ceil(K/256) blocks of 16*pieces*128 code bytes (row 16 p + t = piece p of token t, 16-byte
 * chunk c of row r at c ^ (r & 7)) followed by their 2048-byte scale slab
 * (tpb200_nvfp4_gemv_tc_x_image_bytes), x_row_scale: 16 floats.  Row tiles whose K range is split
 * across CTAs are combined through `workspace` (size from tpb200_nvfp4_gemv_tc_workspace_size; the
 * caller zeroes it ONCE after allocation, the kernel leaves its counters at zero; after a non-zero
 * tpb200_device_error() zero it again before reuse).  Launches that share a workspace must not overlap.
 * The host plans each launch (whole 256-row tiles dealt to the CTAs longest first; tiles are cut along K
 * only when a launch has too few or too long tiles for the machine; a launch that fills the machine several
 * times over leaves a third of its units in a pool that the CTAs draw from as they become free, through one
 * ticket counter in the workspace) and remembers the plans of the last few shape lists per calling thread.  No counterpart in the reference (its GEMVs are CUDA-core kernels).
 *
 * tpb200_nvfp4_gemv_tc_fused is the same GEMV with the activation quantiser inside the launch: `x` is
 * the raw [M, K] activation tensor (x_dtype, row stride ldx elements, 0 = K) and four warps of every CTA
 * quantise the K ranges their CTA needs straight into its stage buffers, so a decode step is ONE launch
 * and there is no activation image in global memory.
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    const void* w_image;
    const void* x_image; const float* x_row_scale;
    const void* bias; void* out;
    int N; int K; int ldo; /* 0 = N */
    float global_scale;
} tpb200_gemv_tc_problem;
size_t tpb200_nvfp4_gemv_tc_workspace_size(const tpb200_gemv_tc_problem* problems, int count);
size_t tpb200_nvfp4_gemv_tc_x_image_bytes(int K, int pieces);
int tpb200_nvfp4_quantize_act_tc(const void* x, int x_dtype, int ldx, void* x_image, float* row_scale, int M, int K,
                                 int pieces, int flags, tpb200_stream_t stream);
/* several activation tensors (different K) of one step in ONE launch */
#define TPB200_MAX_ACTS 8
typedef struct { const void* x; int ldx; int K; void* x_image; float* x_row_scale; } tpb200_act_tc;
int tpb200_nvfp4_quantize_acts_tc(const tpb200_act_tc* acts, int count, int x_dtype, int M, int pieces, int flags,
                                  tpb200_stream_t stream);
int tpb200_nvfp4_gemv_tc(const tpb200_gemv_tc_problem* problems, int count, int M, int pieces, int bias_dtype,
                         int out_dtype, int activation, void* workspace, size_t workspace_bytes, int flags,
                         tpb200_stream_t stream);
typedef struct {
    const void* w_image;
    const void* x; int ldx; /* 0 = K */
    const void* bias; void* out;
    int N; int K; int ldo; /* 0 = N */
    float global_scale;
} tpb200_gemv_tc_fused_problem;
size_t tpb200_nvfp4_gemv_tc_fused_workspace_size(const tpb200_gemv_tc_fused_problem* problems, int count);
int tpb200_nvfp4_gemv_tc_fused(const tpb200_gemv_tc_fused_problem* problems, int count, int M, int pieces, int x_dtype,
                               int bias_dtype, int out_dtype, int activation, void* workspace, size_t workspace_bytes,
                               int flags, tpb200_stream_t stream);

/* What the launch planner does with a list of [N, K] problems on a GPU of `sms` SMs (host only, no device
 * needed): CTAs used, work units, K stages of the busiest CTA and of the whole launch, tiles cut along K,
 * scratch bytes.  For tests and capacity planning. */
typedef struct {
    int grid; int units; int max_load_stages; /* of a CTA's fixed list */ int total_stages; int cut_tiles;
    int pool_units; /* units not tied to a CTA, drawn by whichever CTA is free */ size_t workspace_bytes;
} tpb200_gemv_tc_plan_info;
int tpb200_nvfp4_gemv_tc_plan(const int* N, const int* K, int count, int sms, tpb200_gemv_tc_plan_info* info);

/* tpb200_nvfp4_gemv_tc for callers that cannot allocate device memory (no counterpart in the reference).
 * The split-K scratch is a 4 MiB array built into the library (tpb200_nvfp4_gemv_tc_static_capacity());
 * launches whose plan needs more are refused with TPB200_ERR_WORKSPACE.  The call allocates nothing.
 * The first call on a device looks up the array's device address; make that first call outside of any
 * stream capture.  All calls on a device share the one array: two calls that may run at the same time
 * on the GPU (different streams, different threads) race on it and must be serialised by the caller. */
size_t tpb200_nvfp4_gemv_tc_static_capacity(void);
int tpb200_nvfp4_gemv_tc_static(const tpb200_gemv_tc_problem* problems, int count, int M, int pieces,
                                int bias_dtype, int out_dtype, int activation, int flags, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Attention softmax(scale * Q K^T + key_bias) V on the tensor cores, bf16 in / bf16 out, fp32 softmax.
 * Replaces the scaled_dot_product_attention calls of the reference model
 * (openpi/src/openpi/models_pytorch/pi0_pytorch.py:476-501 prefix, :608-627 / :723-727 action expert;
 * eager forms: transformers_replace/models/gemma/modeling_gemma.py:222-245, .../siglip/modeling_siglip.py:325-345).
 *   q [n_rows, head_dim] (row stride ldq), k / v [n_keys, head_dim], out [n_rows, head_dim]; head_dim a
 *   multiple of 8, <= 256.  Gemma's 8 query heads on one key/value head are passed as n_rows = tokens * 8
 *   rows of the [tokens, 8 * 256] projection (ldq = 256).  groups_outer x groups_inner independent problems
 *   (SigLIP: images x heads) start at base + a * stride[0] + b * stride[1] elements.
 *   key_bias: bf16 [n_keys] added to every row's scores (0, or the mask value for a key that must not be
 *   attended to), NULL = none.
 * Keys are split in tiles of 256 across CTAs; with more than one tile the partial results pass through
 * `workspace` (tpb200_attention_workspace_size bytes, no initialisation needed) and a second small kernel.
 * Group strides are >= 0; a stride of 0 lets every group read the same rows (shared keys / values).
 * ------------------------------------------------------------------------------------------- */
typedef struct {
    const void* q; const void* k; const void* v; void* out; const void* key_bias;
    int n_rows; int n_keys; int head_dim;
    int ldq; int ldk; int ldv; int ldo;
    int groups_outer; int groups_inner;
    long long q_stride[2]; long long k_stride[2]; long long v_stride[2]; long long o_stride[2];
    float scale;
    void* workspace; size_t workspace_bytes;
    int flags;
    /* Optional fused hand-over to the next linear (single problem only, groups 1 x 1): when quant_image is not
     * NULL, every token (= quant_rows_per_token consecutive rows, K = quant_rows_per_token * head_dim, a
     * multiple of 256, <= 8192) is also written as a row of the tiled A image of tpb200_nvfp4_gemm_ex
     * (quant_pieces residual pieces, quant_row_scale[token] = the row multiplier), exactly as
     * tpb200_row_transform_quantize in plain mode would produce from `out`; `out` may then be NULL.  Needs the
     * workspace whatever the key count.
     * quant_sf != NULL selects the GEMM's row-major operand form instead: quant_image = the codes
     * [quant_pieces * quant_piece_rows, quant_pitch] bytes (piece p of token t at row p * quant_piece_rows + t,
     * quant_piece_rows a multiple of 128, quant_pitch >= K / 2 and a multiple of 16), quant_sf = their swizzled
     * scale atoms. */
    void* quant_image; float* quant_row_scale; int quant_pieces; int quant_rows_per_token;
    void* quant_sf; int quant_pitch; int quant_piece_rows;
} tpb200_attention_args;
size_t tpb200_attention_workspace_size(int n_rows, int n_keys, int head_dim, int groups);
int tpb200_attention(const tpb200_attention_args* args, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Row-wise glue between two linears, fused with the activation quantiser of the tensor-core GEMM:
 *   h = res_in + x * gate (optional)  ->  RMSNorm (1 + w0) | adaptive RMSNorm (1 + w0) + w1 | LayerNorm w0, w1
 *   or  GELU_tanh(x[:, :K]) * x[:, K:2K]  |  SiLU(x[:, :K]) * x[:, K:2K]   (gated MLPs)
 * with the roundings of the PyTorch modules (GemmaRMSNorm, _gated_residual, GemmaMLP:
 * openpi/src/openpi/models_pytorch/transformers_replace/models/gemma/modeling_gemma.py:49-129,212-230),
 * written as residual e2m1 pieces + swizzled UE4M3 scales + row multipliers (the A operand of
 * tpb200_nvfp4_gemm_ex), optionally also as bf16 (y_out) and as the updated residual stream (h_out).
 * All tensors bf16, K % 16 == 0, K <= 16384.
 * ------------------------------------------------------------------------------------------- */
enum { TPB200_ROW_NONE = 0, TPB200_ROW_RMSNORM = 1, TPB200_ROW_ADARMS = 2, TPB200_ROW_LAYERNORM = 3,
       TPB200_ROW_GELU_MUL = 4, TPB200_ROW_SILU_MUL = 5 };
typedef struct {
    int mode; int M; int K;
    const void* x; int ldx;
    const void* res_in; const void* gate; void* h_out;
    const void* w0; const void* w1; float eps;
    void* y_out;
    void* packed; int pitch; void* sf; float* row_scale; int pieces; int piece_rows;
    int layout;   /* TPB200_OPERANDS_TILED: `packed` is the GEMM's tiled A image (pitch, sf, piece_rows unused) */
    int flags;    /* TPB200_FLAG_PDL: programmatic stream serialisation, as for the GEMM */
} tpb200_rowop_args;
int tpb200_row_transform_quantize(const tpb200_rowop_args* args, tpb200_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Entry points with the reference's names and signatures (TensorRT-plugin / test ABI).
 * ------------------------------------------------------------------------------------------- */

/* openpi/nvfp4_packed_plugin/src/nvfp4_packed_plugin.h:50-64: block 32, scales in the dtype
 * named by data_type, scale_A may be NULL (weight-only). */
void nvfp4_gemv_forward(const void* activation, const void* weight_packed, const void* scale_A,
                        const void* scale_W, const void* bias, void* output, int M, int N, int K,
                        int activation_type, int data_type, tpb200_stream_t stream);
size_t nvfp4_gemv_workspace_size(int M, int N, int K);

/* openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:61-81: signed int4 (two's complement nibbles, even k
 * in the low nibble) [N, K/2], bf16 scales/zeros [N, K/group]. */
void quantizeWeightToINT4(const void* input_bf16, int8_t* output_packed, void* scales_bf16, void* zeros_bf16,
                          int N, int K, int group_size, tpb200_stream_t stream);
void dequantizeINT4ToBF16(const int8_t* input_packed, const void* scales_bf16, const void* zeros_bf16,
                          void* output_bf16, int N, int K, int group_size, tpb200_stream_t stream);

/* openpi/w4a16_plugin/src/w4a16_gemm_plugin.h:41-59: out bf16 [M,N] = alpha * act bf16 [M,K] @ dequant(W)^T + beta * out,
 * W signed int4 [N, K/2], bf16 scales and optional zero points [N, K/128] (q * scale + zero).  Up to 16 rows run
 * on the decode GEMV (workspace only with zero points or beta != 0), more rows on the tensor-core GEMM of
 * tpb200_w4a16_gemm (no workspace). */
void w4a16GemmForward(const void* activation, const void* weight_packed, const void* weight_scale,
                      const void* weight_zero, void* output, int M, int N, int K, float alpha, float beta,
                      void* workspace, size_t workspaceSize, tpb200_stream_t stream);
size_t getW4A16GemmWorkspaceSize(int M, int N, int K);

/* openpi/w4a8_plugin/src/w4a8_gemm_plugin.h:39-73: out bf16 [M,N] = alpha * (fp8 act * act scale) @ (e2m1 * w scale),
 * weights and their scales stored transposed ([K/2, N], [K/16, N]); N % 8 == 0; the workspace (size from
 * getW4A8GemmWorkspaceSize) holds the re-laid-out operands.  bf16 -> E4M3 values + E4M3 scale per 16 along K;
 * bf16 [N, K] weight -> e2m1 packed TRANSPOSED [K/2, N] + E4M3 scales [K/16, N]. */
void w4a8GemmForward(const void* activation_fp8, const void* activation_scale, const void* weight_packed,
                     const void* weight_scale, void* output_bf16, int M, int N, int K, float alpha, void* workspace,
                     size_t workspaceSize, tpb200_stream_t stream);
size_t getW4A8GemmWorkspaceSize(int M, int N, int K);
void quantizeActivationToFP8(const void* input_bf16, void* output_fp8, void* scales_fp8, int M, int K,
                             tpb200_stream_t stream);
void quantizeWeightToNVFP4(const void* input_bf16, uint8_t* output_packed, void* scales_fp8, int N, int K,
                           tpb200_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOPI_B200_H_ */
