/*
 * gewell_b200 -- C ABI of the B200 (sm_100a) quantised-projection and MoE path.
 *
 * Plain pointers and sizes only.  Every device pointer is a CUDA device
 * address in the current context; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream).  Functions return GW_OK or an error code
 * and leave a message retrievable with gw_last_error() (thread local).
 *
 * "Reference" below means the leDissolution/gewell sources; each entry point
 * names the reference interface it stands in for (path:line in that project).
 *
 * Unless stated otherwise a call neither allocates device memory nor
 * synchronises, and is ordered on `stream` only, so it may be captured in a
 * CUDA graph (plan / workspace construction must happen outside capture).
 */
#ifndef GEWELL_B200_H_
#define GEWELL_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int gw_status;
enum {
  GW_OK = 0,
  GW_INVALID_ARGUMENT = 1, /* contract violation; the reference throws std::invalid_argument */
  GW_CUDA_ERROR = 2,       /* CUDA runtime/driver failure; the reference throws std::runtime_error */
  GW_KERNEL_ERROR = 3,     /* a kernel reported a bounded-wait timeout or internal check */
  GW_UNSUPPORTED = 4       /* valid in the reference, not built here (see message) */
};

/* Message of the last failing call on this host thread ("" if none). */
const char* gw_last_error(void);
/* ABI version of this library (bumped on incompatible change). */
int gw_abi_version(void);

/* ------------------------------------------------------------------------- */
/* Layout helpers -- include/gewell/nvfp4_linear.h:35-56, fp8_linear.h:28-33  */
/* ------------------------------------------------------------------------- */
size_t gw_nvfp4_scale_storage_bytes(size_t rows, size_t input_width);
size_t gw_nvfp4_scale_offset(size_t row, size_t block, size_t input_width);
size_t gw_nvfp4_scratch_upper_bound_bytes(size_t max_rows, size_t input_width, size_t output_width);
size_t gw_fp8_scratch_upper_bound_bytes(size_t max_rows, size_t input_width);

enum { GW_TRANSFORM_IDENTITY = 0, GW_TRANSFORM_GELU_TANH_MULTIPLY = 1 };

/* ------------------------------------------------------------------------- */
/* NVFP4                                                                      */
/* ------------------------------------------------------------------------- */

/* gewell::nvfp4::dequantize (include/gewell/nvfp4_linear.h:28-33,
 * src/nvfp4_linear.cu:39-56,120-132): packed E2M1 [N,K/2] + tiled E4M3 scales
 * -> row-major BF16 [N,K] = bf16(e2m1 * (e4m3 * weight_scale)).
 * K % 64 == 0, N % 128 == 0, weight_scale finite and > 0. */
gw_status gw_nvfp4_dequantize(const uint8_t* data, const uint8_t* scales, float weight_scale,
                              uint32_t input_width, uint32_t output_width, void* output_bf16,
                              void* stream);

/* Device weight packer: the recipe of tools/convert.py:111-137
 * (quantize_nvfp4_tensor) and src/weight_qdq_detail.cuh:73-82 applied to a
 * BF16 matrix [N,K] with a caller-supplied global weight_scale
 * (= amax/(6*448), see gw_absmax_bf16).  Writes packed [N,K/2] and tiled scale
 * storage (gw_nvfp4_scale_storage_bytes(N,K) bytes, padding zeroed). */
gw_status gw_nvfp4_pack_weights(const void* weights_bf16, uint32_t output_width, uint32_t input_width,
                                float weight_scale, uint8_t* data, uint8_t* scales, void* stream);

/* Activation quantiser of nvfp4::Plan::run (src/nvfp4_linear.cu:61-116),
 * exposed for tests: BF16 [rows,K] (or [rows,2K] gate|up with the GeGLU
 * transform) -> packed [rows,K/2] + tiled scales for `rows` rows. */
gw_status gw_nvfp4_quantize_activations(const void* input_bf16, uint32_t rows, uint32_t input_width,
                                        float input_scale, int transform, uint8_t* packed,
                                        uint8_t* scales, void* stream);

/* gewell::nvfp4::Plan (include/gewell/nvfp4_linear.h:64-91,
 * src/nvfp4_linear.cu:134-330).  Y[rows,N] = bf16(alpha * Xq . Wq^T),
 * alpha = input_scale*weight_scale, tcgen05 block-scaled MMA.  The cuBLASLt
 * handle of the reference constructor has no counterpart (no library GEMM). */
typedef struct gw_nvfp4_plan gw_nvfp4_plan;
gw_status gw_nvfp4_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width,
                               gw_nvfp4_plan** plan);
size_t gw_nvfp4_plan_scratch_bytes(const gw_nvfp4_plan* plan);
gw_status gw_nvfp4_plan_run(gw_nvfp4_plan* plan, const void* input_bf16, const uint8_t* weight_data,
                            const uint8_t* weight_scales, float input_scale, float weight_scale,
                            void* output_bf16, void* scratch, size_t scratch_capacity, void* stream,
                            int transform);
void gw_nvfp4_plan_destroy(gw_nvfp4_plan* plan);

/* NVFP4 linear layer for callers that cannot allocate device memory and have
 * no scratch region to lend (no counterpart in the reference, whose Plan::run
 * always takes caller scratch).  Same arithmetic and kernels as
 * gw_nvfp4_plan_run, but the packed activations and their scale tiles go to a
 * fixed array built into this library, so the call takes inputs and outputs
 * only and performs no allocation of any kind.
 *   - limit: rows*K/2 (rounded up to 256) + gw_nvfp4_scale_storage_bytes(rows,K)
 *     must not exceed gw_nvfp4_linear_static_scratch_limit() (2 MiB); larger
 *     problems are rejected with GW_INVALID_ARGUMENT;
 *   - the array is resident on every GPU that loads the library, for the
 *     lifetime of the process;
 *   - the first call on each GPU looks up the array's device address; make
 *     that first call before starting any stream capture;
 *   - all calls on a GPU share the array: calls that overlap on the GPU
 *     (several streams or host threads) race -- keep them on one stream. */
size_t gw_nvfp4_linear_static_scratch_limit(void);
gw_status gw_nvfp4_linear_static_scratch(const void* input_bf16, uint32_t rows, uint32_t input_width,
                                         uint32_t output_width, const uint8_t* weight_data,
                                         const uint8_t* weight_scales, float input_scale, float weight_scale,
                                         void* output_bf16, void* stream, int transform);

/* W4A16 projection (models/gemma4/26b_a4b/sm120/projection.cu:129-139 and the
 * north-star host path): BF16 activations times NVFP4 weights without
 * activation quantisation, for small row counts; weights are streamed once
 * and decoded in registers.  rows <= 8. */
gw_status gw_nvfp4_gemv_w4a16(const void* input_bf16, uint32_t rows, const uint8_t* weight_data,
                              const uint8_t* weight_scales, float weight_scale, uint32_t input_width,
                              uint32_t output_width, void* output_bf16, void* stream);

/* ------------------------------------------------------------------------- */
/* FP8                                                                        */
/* ------------------------------------------------------------------------- */

/* Activation quantiser of fp8::Plan::run (src/fp8_linear.cu:33-52). */
gw_status gw_fp8_quantize_activations(const void* input_bf16, uint32_t rows, uint32_t input_width,
                                      float input_scale, int transform, uint8_t* packed, void* stream);

/* Device E4M3 weight packer: tools/convert.py:49-62 with a caller-supplied
 * scalar scale, or one scale per output row when row_scales != NULL. */
gw_status gw_fp8_pack_weights(const void* weights_bf16, uint32_t output_width, uint32_t input_width,
                              float weight_scale, const float* row_scales, uint8_t* data, void* stream);

/* gewell::fp8::Plan (include/gewell/fp8_linear.h:40-69, src/fp8_linear.cu:56-271)
 * including the per-output-channel ("joined") variant that the reference
 * serves with fp8::detail::ScaledGemm (src/fp8_scaled_gemm.cuh:18-97). */
typedef struct gw_fp8_plan gw_fp8_plan;
gw_status gw_fp8_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width,
                             int channel_scales, gw_fp8_plan** plan);
size_t gw_fp8_plan_scratch_bytes(const gw_fp8_plan* plan);
gw_status gw_fp8_plan_run(gw_fp8_plan* plan, const void* input_bf16, const uint8_t* weight_data,
                          float input_scale, float weight_scale, const float* channel_scales,
                          void* output_bf16, void* scratch, size_t scratch_capacity, void* stream,
                          int transform);
void gw_fp8_plan_destroy(gw_fp8_plan* plan);

/* ------------------------------------------------------------------------- */
/* BF16                                                                       */
/* ------------------------------------------------------------------------- */

/* BF16 linear layer Y[rows,N] = bf16(X . W^T), FP32 accumulation on tcgen05 kind::f16: the role of
 * the reference's BF16 LinearPlan (models/gemma4/31b/sm120/resources.cuh:118) and of the
 * cublasGemmEx call of its W4A16 / BF16 projection path (models/gemma4/26b_a4b/sm120/projection.cu:
 * 130-139).  K and N divisible by 8; X [rows,K], W [N,K], Y [rows,N] row-major BF16, 16-byte aligned.
 * scratch: gw_bf16_plan_scratch_bytes() bytes, 256-byte aligned (FP32 partial tiles of the K split
 * that decode-shaped plans use), or NULL to run without the split. */
typedef struct gw_bf16_plan gw_bf16_plan;
gw_status gw_bf16_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width, gw_bf16_plan** plan);
size_t gw_bf16_plan_scratch_bytes(const gw_bf16_plan* plan);
gw_status gw_bf16_plan_run(gw_bf16_plan* plan, const void* input_bf16, const void* weight_bf16, void* output_bf16,
                           void* scratch, size_t scratch_capacity, void* stream);
void gw_bf16_plan_destroy(gw_bf16_plan* plan);

/* ------------------------------------------------------------------------- */
/* Weight QDQ -- src/weight_qdq.cu:105-189,222-258 (detail::apply_tensor)     */
/* ------------------------------------------------------------------------- */
enum { GW_QDQ_BF16 = 0, GW_QDQ_FP8 = 1, GW_QDQ_NVFP4 = 2 };

/* |x| maximum of a BF16 tensor and a non-finite flag, as
 * accumulate_absmax_kernel (src/weight_qdq.cu:105-148).  state = two uint32
 * on the device {float bits of amax, nonfinite flag}; cleared by this call. */
gw_status gw_absmax_bf16(const void* values_bf16, uint64_t elements, uint32_t* state, void* stream);

/* In-place BF16 -> grid -> BF16 fake quantisation of one tensor.  Like the
 * reference this reads the maximum back to the host, so it SYNCHRONISES the
 * stream; non-finite input is rejected (GW_INVALID_ARGUMENT).  `state` as above. */
gw_status gw_weight_qdq_apply(int type, void* values_bf16, uint64_t elements, uint32_t* state,
                              void* stream);

/* ------------------------------------------------------------------------- */
/* MoE -- models/gemma4/26b_a4b/sm120/{projection.cuh:11-17, moe.cuh:11-48}   */
/* ------------------------------------------------------------------------- */
enum { GW_STORAGE_BF16 = 0, GW_STORAGE_NVFP4_W4A4 = 1, GW_STORAGE_FP8_W8A8 = 2,
       /* expert-parallel only (no counterpart in the reference): the expert's
        * weights live on another rank; all three projections carry this tag */
       GW_STORAGE_ABSENT = 3 };

/* sm120::Projection (projection.cuh:11-17), flattened. */
typedef struct gw_projection {
  uint32_t storage;
  uint32_t input, output, physical_output;
  const void* bf16;
  const uint8_t* nvfp4_data;   /* [physical_output, input/2], padding rows zero */
  const uint8_t* nvfp4_scales; /* tiled, padding zero */
  float nvfp4_input_scale, nvfp4_weight_scale;
  const uint8_t* fp8_data;
  float fp8_input_scale, fp8_weight_scale;
  const float* fp8_channel_scales;
} gw_projection;

/* sm120::ExpertWeights (moe.cuh:11-13). */
typedef struct gw_expert_weights {
  gw_projection gate, up, down;
} gw_expert_weights;

/* nvfp4::ActivationPolicy / nvfp4::Phase / fp4_activations (include/gewell/nvfp4_policy.h:7-12):
 * policy "prefill" keeps decode activations in BF16 (NVFP4 weights are then used as W4A16). */
enum { GW_POLICY_ALWAYS = 0, GW_POLICY_PREFILL = 1 };
enum { GW_PHASE_PREFILL = 0, GW_PHASE_DECODE = 1 };
int gw_nvfp4_fp4_activations(int policy, int phase);

/* bind_projection (projection.cu:31-50): describe one artifact entry as a projection.  The entry is
 * `rows` x `columns` (output x input) in `storage`; its payload starts at host_payload /
 * device_payload (the same bytes on both sides) and is entry_bytes long:
 *   BF16   [rows, columns] BF16
 *   FP8    [rows, columns] E4M3, then <f32 weight_scale><f32 input_scale>
 *   NVFP4  [rows padded to 128, columns/2] packed E2M1 (padding rows zero), tiled E4M3 scales for the
 *          padded rows (padding zero), then <f32 weight_scale><f32 input_scale>
 * with the two globals in the entry's last eight bytes (little endian).  Host-only; no device access. */
gw_status gw_bind_projection(uint32_t storage, uint32_t rows, uint32_t columns, const uint8_t* host_payload,
                             const void* device_payload, size_t entry_bytes, gw_projection* projection);

/* Size and content checks of one artifact entry before it is bound, as the reference's artifact reader
 * applies them to every projection (models/gemma4/26b_a4b/artifact.cc:64-104): the entry's byte count
 * for its shape and storage, finite positive global scales with a finite reciprocal and product, no
 * NaN codes in FP8 payloads, zero padding rows and zero padding scales in NVFP4 payloads, block scale
 * codes below 0x7f.  Host-only.  (The file container around the entries -- header, entry table,
 * SHA-256 digests -- is not read here.) */
size_t gw_projection_entry_bytes(uint32_t storage, uint32_t rows, uint32_t columns);
gw_status gw_validate_projection_entry(uint32_t storage, uint32_t rows, uint32_t columns, const uint8_t* host_payload,
                                       size_t entry_bytes);

/* The artifact container itself (G4A4MIX1 / G4A4BF16): ArtifactFile of the reference
 * (include/gewell/models/gemma4/26b_a4b/artifact.h, src/models/gemma4/26b_a4b/artifact.cc:105-221).
 * gw_artifact_open memory-maps the file and checks, like ArtifactFile::Open / ValidateMetadata:
 * identity, the ten geometry fields, the tied-head alias, reserved bytes, the SHA-256 of the header
 * and of the entry table, every 72-byte entry against the inventory (id, layer, role, rank, shape,
 * running offset, byte count for its storage type), the five size fields against the file's length,
 * and the global scales of every quantised entry.  gw_artifact_verify_full is VerifyFull: table
 * padding, every payload (gw_validate_projection_entry), per-tensor and whole-payload SHA-256, zero
 * padding between tensors.  The reference compiles the model's tensor inventory into the reader; here
 * the caller passes it (one spec per physical tensor, in file order; `projection` != 0 marks the
 * tensors that may be stored quantised; `columns` is ignored for rank 1).  Host code only; entry.data
 * points into the mapping and is valid until gw_artifact_close. */
typedef struct gw_artifact_tensor_spec {
  int32_t layer;
  uint32_t role, rank, rows, columns, projection;
} gw_artifact_tensor_spec;
typedef struct gw_artifact_entry {
  uint64_t offset, bytes;
  uint32_t storage;
  uint8_t sha256[32];
  const uint8_t* data;
} gw_artifact_entry;
typedef struct gw_artifact gw_artifact;
gw_status gw_artifact_open(const char* path, const gw_artifact_tensor_spec* inventory, uint32_t count,
                           gw_artifact** artifact);
uint32_t gw_artifact_count(const gw_artifact* artifact);
int gw_artifact_is_mixed(const gw_artifact* artifact);
uint64_t gw_artifact_file_bytes(const gw_artifact* artifact);
gw_status gw_artifact_entry_at(const gw_artifact* artifact, uint32_t id, gw_artifact_entry* entry);
gw_status gw_artifact_verify_full(const gw_artifact* artifact);
void gw_artifact_close(gw_artifact* artifact);

/* ProjectionWorkspace (projection.cuh:19-41, projection.cu:52-145): shared scratch and plans for
 * sequential projections on ONE stream, bound at construction.  create() sizes the scratch for
 * max_rows and the given bindings and allocates it; prepare(rows, phase) builds the plans for a row
 * count before the layer loop (it allocates small per-plan state: not capturable); run() allocates
 * nothing and picks the path by storage, policy and phase (W8A8, W4A4, or BF16 GEMM on BF16 weights /
 * on the NVFP4 weight dequantised to BF16), then strips NVFP4 output padding.  The reference's
 * cublasHandle_t argument of run has no counterpart (no library GEMM). */
typedef struct gw_projection_workspace gw_projection_workspace;
gw_status gw_projection_workspace_create(const gw_projection* projections, uint32_t count, uint32_t max_rows,
                                         int policy, void* stream, gw_projection_workspace** workspace);
gw_status gw_projection_workspace_prepare(gw_projection_workspace* workspace, uint32_t rows, int phase);
gw_status gw_projection_workspace_run(gw_projection_workspace* workspace, const gw_projection* projection,
                                      const void* input_bf16, void* output_bf16);
size_t gw_projection_workspace_bytes(const gw_projection_workspace* workspace);
void gw_projection_workspace_destroy(gw_projection_workspace* workspace);

/* ------------------------------------------------------------------------- */
/* Dense MLP chain of the 31B model                                           */
/* ------------------------------------------------------------------------- */

/* GeGLU with both BF16 roundings (src/bf16_activation.cuh:10-16) as stand-alone kernels: on separate
 * gate / up arrays, and on a joined [rows, gate | up] tensor (primitives::gelu_tanh_multiply and
 * gelu_tanh_multiply_interleaved of the 31B executor). */
gw_status gw_gelu_tanh_multiply_bf16(const void* gate_bf16, const void* up_bf16, void* output_bf16, uint64_t count,
                                     void* stream);
gw_status gw_gelu_tanh_multiply_interleaved_bf16(const void* gate_up_bf16, void* output_bf16, uint32_t rows,
                                                 uint32_t width, void* stream);

/* Executor::project_mlp with projection_linear (models/gemma4/31b/sm120/executor.cuh:1187-1215,
 * 1248-1291): gate + up projection -> GeGLU -> down projection of one layer, from the layer's three
 * bound weights (gw_projection: BF16, FP8 or NVFP4 each; physical_output == output).  Gate and up run
 * as ONE GEMM when they are stored back to back (NVFP4: contiguous rows and scale tiles with equal
 * globals, 31b/sm120/nvfp4_projections.h:21-33; FP8: adjacent with per-channel scales,
 * fp8_projections.h:20-50; BF16: adjacent); GeGLU is fused into the down projection's activation
 * quantiser whenever that one runs quantised on the joined tensor.  policy / phase as in
 * nvfp4_policy.h: with policy "prefill" decode keeps BF16 activations (NVFP4 weights are dequantised
 * into the chain's scratch, W4A16).
 *   create    allocates the shared scratch for max_rows (set-up time)
 *   prepare   builds the plans for a row count, outside the layer loop
 *   run       gate_up_bf16: [rows, 2 * mlp] scratch of the caller ([rows, gate | up] when joined, gate
 *             rows then up rows otherwise), product_bf16: [rows, mlp] scratch (used by the unfused
 *             GeGLU), output_bf16: [rows, hidden]; allocates nothing */
typedef struct gw_mlp_chain gw_mlp_chain;
gw_status gw_mlp_chain_create(uint32_t hidden, uint32_t mlp, uint32_t max_rows, int policy, gw_mlp_chain** chain);
gw_status gw_mlp_chain_prepare(gw_mlp_chain* chain, uint32_t rows);
gw_status gw_mlp_chain_run(gw_mlp_chain* chain, const gw_projection* gate, const gw_projection* up,
                           const gw_projection* down, const void* input_bf16, void* gate_up_bf16, void* product_bf16,
                           void* output_bf16, int phase, void* stream);
size_t gw_mlp_chain_bytes(const gw_mlp_chain* chain);
void gw_mlp_chain_destroy(gw_mlp_chain* chain);

/* Executor::project_qkv without its norms (models/gemma4/31b/sm120/executor.cuh:1218-1247): the
 * attention input projections of one layer.  One joined GEMM when Q, K (and V) are adjacent BF16
 * matrices (fusion::qkv_weight, projection_fusion.h:23-33) or adjacent FP8 matrices with adjacent
 * per-channel scales and one input scale (fp8::qkv_weight, fp8_projections.h:26-35): *joined = 1 and
 * q_bf16 receives [rows, Q | K | V]; otherwise *joined = 0 and every projection writes its own output
 * (FP8 -> NVFP4 with FP4 activations -> BF16 GEMM, as projection_linear :1187-1215).  `value` NULL for
 * layers whose values are their keys (global attention).  Widths divisible by 128. */
typedef struct gw_qkv_projector gw_qkv_projector;
gw_status gw_qkv_projector_create(uint32_t hidden, uint32_t q_width, uint32_t kv_width, uint32_t max_rows, int policy,
                                  gw_qkv_projector** projector);
gw_status gw_qkv_projector_prepare(gw_qkv_projector* projector, uint32_t rows);
gw_status gw_qkv_projector_run(gw_qkv_projector* projector, const gw_projection* query, const gw_projection* key,
                               const gw_projection* value, const void* input_bf16, void* q_bf16, void* k_bf16,
                               void* v_bf16, int phase, void* stream, int* joined);
size_t gw_qkv_projector_bytes(const gw_qkv_projector* projector);
void gw_qkv_projector_destroy(gw_qkv_projector* projector);

/* The joins the 31B loader makes in place after uploading a layer (Weights, weights.cuh:146-223), so
 * that the joined forms above apply.  Both rewrite device memory on `stream` and update the
 * projections' pointers; *joined = 0 and nothing changes when the group does not qualify.
 *   gw_join_nvfp4_pair: two NVFP4 matrices of one shape with equal input and weight scales, the
 *     second payload somewhere behind the first in one region -> [first rows | second rows | first
 *     scale tiles | second scale tiles] from the first matrix's address on.  temp: 2 * (packed +
 *     scale) bytes of device memory.
 *   gw_join_fp8_group: FP8 matrices with one input scale and one K, in ascending address order ->
 *     their rows packed back to back from the first matrix's address on, channel_scales (device,
 *     one float per output channel of the group) filled with input_scale * weight_scale of each
 *     channel's own matrix.  temp: the group's weight bytes.  Synchronises the stream. */
gw_status gw_join_nvfp4_pair(gw_projection* first, gw_projection* second, void* temp, size_t temp_bytes, void* stream,
                             int* joined);
gw_status gw_join_fp8_group(gw_projection* group, uint32_t count, float* channel_scales, void* temp, size_t temp_bytes,
                            void* stream, int* joined);

/* The reference keeps the 128-entry ExpertWeights table in device memory and
 * reads it from its kernels (batched_executor.cu:62-88).  Here the table is
 * bound once from the host copy: the call validates it, builds the TMA
 * descriptors of every expert matrix and uploads both.  Allocates; not
 * capturable.  `experts` has `count` (=128) entries in host memory. */
typedef struct gw_expert_table gw_expert_table;
gw_status gw_moe_expert_table_create(const gw_expert_weights* experts, uint32_t count,
                                     gw_expert_table** table);
void gw_moe_expert_table_destroy(gw_expert_table* table);
/* Every projection may have its own storage type (BF16, FP8 W8A8, NVFP4), as in the reference.
 * NVFP4 experts used with BF16 activations (fp4 == 0 in gw_moe_run: the reference's grouped_linear,
 * moe.cu:96-103,353-395, which decodes weight tiles to BF16 in shared memory) run here on BF16 copies
 * of their weights, made once by this call (allocates 2 bytes per weight and dequantises on `stream`,
 * then synchronises it): set-up time, not capturable.  Without it gw_moe_run(fp4 == 0) returns
 * GW_UNSUPPORTED for NVFP4 experts. */
gw_status gw_moe_expert_table_enable_w4a16(gw_expert_table* table, void* stream);

/* sm120::MoeWorkspace (moe.cuh:20-48, moe.cu:462-545).  max_rows in 1..65536
 * (the reference stops at 4096).  All buffers are allocated here, once. */
typedef struct gw_moe_workspace gw_moe_workspace;
gw_status gw_moe_create(uint32_t max_rows, gw_moe_workspace** workspace);
/* The same with options.  GW_MOE_FP8_EXPERTS: also allocate the E4M3 staging of FP8 experts' inputs
 * (24 KB per routed token), which the reference's grouped_fp8 (moe.cu:187-251) quantises in registers
 * instead; without it gw_moe_run(has_fp8) returns GW_UNSUPPORTED for tables with FP8 experts. */
enum { GW_MOE_FP8_EXPERTS = 1 };
gw_status gw_moe_create_ex(uint32_t max_rows, uint32_t flags, gw_moe_workspace** workspace);
void gw_moe_destroy(gw_moe_workspace* workspace);

/* MoeWorkspace::dispatch (moe.cu:477-488): routing, stable sort by expert,
 * offsets, inverse permutation.  rows == 0 is a no-op. */
gw_status gw_moe_dispatch(gw_moe_workspace* workspace, const void* scores_bf16,
                          const void* expert_scales_bf16, uint32_t rows, void* stream);

/* MoeWorkspace::run (moe.cu:489-534).  has_bf16 / has_fp8 / has_nvfp4 say which kinds of expert
 * weights the table holds (a kind whose flag is 0 is not computed, as in the reference); fp4 != 0 runs
 * NVFP4 experts with FP4 activations (W4A4), fp4 == 0 with BF16 activations (W4A16, see
 * gw_moe_expert_table_enable_w4a16).  A table of NVFP4 experts only with fp4 != 0 takes the fused
 * large-batch path; every other combination runs one grouped gate/up and down GEMM per kind present
 * (tcgen05 kind::mxf4nvf4 / kind::f16 / kind::f8f6f4) with GeGLU unfused. */
gw_status gw_moe_run(gw_moe_workspace* workspace, const void* input_bf16, const void* scores_bf16,
                     const void* expert_scales_bf16, const gw_expert_table* table, void* output_bf16,
                     uint32_t rows, int has_bf16, int has_fp8, int has_nvfp4, int fp4, void* stream);

/* Accessors of the reference workspace (moe.cuh:29-40, moe.cu:541-544);
 * device pointers valid after the stream has reached the end of run/dispatch. */
const int32_t* gw_moe_selected_experts(const gw_moe_workspace* workspace);   /* [8*rows] ascending per token */
const float* gw_moe_routing_weights(const gw_moe_workspace* workspace);      /* [8*rows] */
const int32_t* gw_moe_offsets(const gw_moe_workspace* workspace);            /* [129] */
const int32_t* gw_moe_sorted_assignments(const gw_moe_workspace* workspace); /* [8*rows] */
/* inverse[8*t + slot] = sorted position of that assignment (moe.cu:158-182 `invert`);
 * the reference keeps it private, the expert-parallel combine needs it. */
const int32_t* gw_moe_inverse(const gw_moe_workspace* workspace);            /* [8*rows] */
const void* gw_moe_gate_up_capture(const gw_moe_workspace* workspace);       /* BF16 [8*rows,1408] */
const void* gw_moe_activated_capture(const gw_moe_workspace* workspace);     /* BF16 [8*rows,704] */
const void* gw_moe_down_capture(const gw_moe_workspace* workspace);          /* BF16 [8*rows,2816] */
size_t gw_moe_bytes(const gw_moe_workspace* workspace);
size_t gw_moe_routing_bytes(const gw_moe_workspace* workspace);
size_t gw_moe_projection_bytes(const gw_moe_workspace* workspace);
size_t gw_moe_reduction_bytes(const gw_moe_workspace* workspace);

/* The reference always materialises the BF16 gate/up and activated
 * intermediates that its capture accessors expose (moe.cuh:38-40).  Large
 * batches here fuse GeGLU and the FP4 quantisation of the down input into the
 * gate/up GEMM and skip those buffers; enable capture to have them written as
 * well (the down capture is always valid).  Off by default. */
gw_status gw_moe_capture(gw_moe_workspace* workspace, int enable);

/* Optional per-stage timing of gw_moe_run (no counterpart in the reference;
 * its backends time whole steps with CUDA events, runtime/backend.h:127-129).
 * When enabled, run records CUDA events on its stream between the stages
 *   0 routing+permutation, 1 group descriptors + gather/quantise,
 *   2 grouped gate/up GEMM, 3 GeGLU + quantise, 4 grouped down GEMM, 5 combine;
 * gw_moe_stage_elapsed_ms waits for the last run and writes six durations. */
gw_status gw_moe_stage_timing(gw_moe_workspace* workspace, int enable);
gw_status gw_moe_stage_elapsed_ms(gw_moe_workspace* workspace, float* milliseconds);

/* ------------------------------------------------------------------------- */
/* Feed-forward block of a 26B-A4B layer around the MoE                       */
/* ------------------------------------------------------------------------- */

/* bf16_math::normalize (bf16_math.cuh:96-98): y[r, c] = bf16(x[r, c] * rsqrt(mean(x[r]^2) + 1e-6) *
 * weight[c]) for `rows` rows of `width` BF16 values (weight NULL: no weight).  The FP32 mean is
 * accumulated in the reference's fixed order, which depends on rows and width (four accumulators per
 * logical lane, lanes folded in a halving tree, normalize_to :86-95), without fused multiply-add.
 * width divisible by 8, at most 16384; x 16-byte aligned. */
gw_status gw_rms_norm_bf16(const void* input_bf16, const void* weight_bf16, void* output_bf16, uint32_t rows,
                           uint32_t width, void* stream);
/* bf16_math::normalize_feedforward (bf16_math.cuh:25-37,99-104): one RMS of the hidden state, three
 * outputs -- shared = bf16(n * shared_weight), expert = bf16(n * expert_weight), and the router input
 * bf16(bf16(bf16(n) * router_weight) / sqrt(width)) with its three separate roundings. */
gw_status gw_rms_norm_feedforward_bf16(const void* input_bf16, const void* shared_weight, const void* router_weight,
                                       const void* expert_weight, void* shared_bf16, void* router_bf16,
                                       void* expert_bf16, uint32_t rows, uint32_t width, void* stream);
/* bf16_math::add (bf16_math.cuh:109-112) and row_scale (batched_executor.cu:30-33). */
gw_status gw_add_bf16(const void* a_bf16, const void* b_bf16, void* output_bf16, uint64_t count, void* stream);
gw_status gw_scale_bf16(void* values_bf16, const void* scalar_bf16, uint64_t count, void* stream);
/* The end of the block in one launch (seven in the reference, batched_executor.cu:260,278-285):
 *   shared = norm(shared_mlp, norm_shared_weight); branch = norm(routed, norm_routed_weight);
 *   shared = bf16(shared + branch); branch = norm(shared, norm_sum_weight);
 *   hidden = bf16(hidden + branch); hidden = bf16(hidden * layer_scalar[0]).
 * Bit-identical to the seven calls above composed. */
gw_status gw_ffn_tail_bf16(const void* shared_mlp_bf16, const void* routed_bf16, const void* norm_shared_weight,
                           const void* norm_routed_weight, const void* norm_sum_weight, const void* layer_scalar_bf16,
                           void* hidden_bf16, uint32_t rows, uint32_t width, void* stream);

/* One layer's feed-forward weights: TensorRole pre_feedforward_norm, router_scale,
 * pre_feedforward_norm_2, post_feedforward_norm_1/_2, post_feedforward_norm, layer_scalar, gate_proj /
 * up_proj / down_proj (shared MLP, 2816 -> 2112 -> 2816), router_proj, router_per_expert_scale and
 * the expert table (include/gewell/models/gemma4/26b_a4b/model.h:38-45,88-105).  Norm weights BF16 [2816],
 * layer_scalar BF16 [1], router_proj BF16 [128, 2816], router_per_expert_scale BF16 [128]: device. */
typedef struct gw_ffn_block_weights {
  const void *pre_feedforward_norm, *router_scale, *pre_feedforward_norm_2;
  const void *post_feedforward_norm_1, *post_feedforward_norm_2, *post_feedforward_norm, *layer_scalar;
  gw_projection gate, up, down;
  const void* router_proj;
  const void* router_per_expert_scale;
  const gw_expert_table* experts;
  int has_bf16, has_fp8, has_nvfp4;
} gw_ffn_block_weights;

/* The block's state for up to max_rows rows: projection workspace over the `count` layers' shared-MLP
 * and router projections, MoE workspace (moe_flags as gw_moe_create_ex) and the intermediate buffers.
 * prepare(rows, phase) builds the plans outside the layer loop; run() applies one layer's block to
 * hidden [rows, 2816] in place on the stream given at creation and allocates nothing
 * (batched_executor.cu:250-286). */
typedef struct gw_ffn_block gw_ffn_block;
gw_status gw_ffn_block_create(const gw_ffn_block_weights* layers, uint32_t count, uint32_t max_rows, int policy,
                              uint32_t moe_flags, void* stream, gw_ffn_block** block);
gw_status gw_ffn_block_prepare(gw_ffn_block* block, uint32_t rows, int phase);
gw_status gw_ffn_block_run(gw_ffn_block* block, const gw_ffn_block_weights* weights, void* hidden_bf16);
size_t gw_ffn_block_bytes(const gw_ffn_block* block);
void gw_ffn_block_destroy(gw_ffn_block* block);
/* Intermediates of the last run (the tensors the reference's capture sink names), device pointers. */
enum { GW_FFN_NORMALIZED = 0, GW_FFN_ROUTER_INPUT = 1, GW_FFN_EXPERT_INPUT = 2, GW_FFN_SHARED_MLP = 3,
       GW_FFN_ROUTER_LOGITS = 4, GW_FFN_ROUTED = 5 };
const void* gw_ffn_block_buffer(const gw_ffn_block* block, int which);
gw_moe_workspace* gw_ffn_block_moe(gw_ffn_block* block);

/* MoE passes over HOST buffers (no counterpart in the reference, whose callers keep activations on
 * the device): for a caller whose token rows, router logits and layer output live in pinned host
 * memory.  The runner owns three streams and a ring of `depth` device buffers; submit() queues
 * upload -> gw_moe_run -> download and returns at once, so the copies of neighbouring passes
 * overlap the kernels.  Results equal gw_moe_run on device buffers bit for bit.
 *   - create/destroy allocate and free device memory (set-up time, not capturable);
 *   - the workspace, the expert table, the weights and `expert_scales_bf16` (device, 128 BF16)
 *     must be complete on the device before the first submit, and the workspace must not be used
 *     by other calls while passes are in flight;
 *   - host_x [rows, 2816], host_scores [rows, 128], host_y [rows, 2816] are BF16 in pinned host
 *     memory (pageable memory works but serialises the copies); host_y is readable after wait()
 *     on the pass's ticket or after synchronize();
 *   - NVFP4 experts with FP4 activations (the mode gw_moe_run is built for). */
typedef struct gw_moe_host_runner gw_moe_host_runner;
gw_status gw_moe_host_runner_create(gw_moe_workspace* workspace, const gw_expert_table* table,
                                    const void* expert_scales_bf16, uint32_t max_rows, uint32_t depth,
                                    gw_moe_host_runner** runner);
void gw_moe_host_runner_destroy(gw_moe_host_runner* runner);
gw_status gw_moe_host_runner_submit(gw_moe_host_runner* runner, const void* host_x, const void* host_scores,
                                    void* host_y, uint32_t rows, uint64_t* ticket);
gw_status gw_moe_host_runner_wait(gw_moe_host_runner* runner, uint64_t ticket);
gw_status gw_moe_host_runner_synchronize(gw_moe_host_runner* runner);
/* The runner's streams (cudaStream_t as void*), e.g. to record timing events around a batch of passes. */
gw_status gw_moe_host_runner_streams(gw_moe_host_runner* runner, void** upload, void** compute, void** download);
/* Bytes copied so far in each direction. */
uint64_t gw_moe_host_runner_h2d_bytes(const gw_moe_host_runner* runner);
uint64_t gw_moe_host_runner_d2h_bytes(const gw_moe_host_runner* runner);

/* Expert-parallel building blocks (no counterpart in the reference, which is
 * single GPU).  A rank that owns experts [first, first+count) runs the expert
 * MLP over rows that are already sorted by expert: `offsets` (device, int32,
 * count+1 entries) delimit each local expert's rows; sorted row i is row
 * row_index[i] of `input_bf16` (row i itself when row_index is NULL); output
 * BF16 [total_rows, 2816] in sorted order, unweighted. */
gw_status gw_moe_run_sorted(gw_moe_workspace* workspace, const void* input_bf16,
                            const int32_t* row_index, const int32_t* offsets, uint32_t first_expert, uint32_t expert_count,
                            uint32_t total_rows, const gw_expert_table* table, void* output_bf16,
                            void* stream);

/* Gather rows by an index vector: out[i,:] = in[index[i] / divisor, :]. */
gw_status gw_gather_rows_bf16(const void* input_bf16, const int32_t* index, uint32_t divisor,
                              uint32_t rows, uint32_t width, void* output_bf16, void* stream);

/* MoeWorkspace reduce step alone (moe.cu:446-456) over caller buffers:
 * out[t,:] = ordered BF16 fold over the 8 slots of down[inverse[8t+j],:]*w[8t+j]. */
gw_status gw_moe_combine(const void* down_bf16, const int32_t* inverse, const float* weights,
                         uint32_t rows, uint32_t width, void* output_bf16, void* stream);

/* Expert parallelism over peer memory (no counterpart in the reference).  Rows
 * travel as 1584-byte records: 1408 bytes of packed E2M1 followed by the row's
 * 176 E4M3 block scales in K order.
 *
 * Buffers that other ranks (processes) of the same node write or read are
 * allocated with gw_ipc_alloc, which also returns a 64-byte handle; a peer turns
 * the handle into a pointer valid in its own process with gw_ipc_open.  Neither
 * call is capturable; both belong to set-up. */
#define GW_IPC_HANDLE_BYTES 64
gw_status gw_ipc_alloc(size_t bytes, void** pointer, uint8_t* handle);
gw_status gw_ipc_open(const uint8_t* handle, void** pointer);
gw_status gw_ipc_close(void* pointer);
gw_status gw_ipc_free(void* pointer);

/* After gw_moe_dispatch on `workspace`: quantise every routed row with its
 * expert's input scale (inverse_input_scales[e] = 1 / input_scale of expert e,
 * 128 floats on the device) and store its record at row
 *   dest_row0[e] + (position of the row among this rank's rows of expert e)
 * of peer_records[dest_rank[e]].  dest_rank / dest_row0: 128 int32 each on the
 * device; peer_records: one device pointer per rank, in device memory, each
 * 16-byte aligned (a record travels as one 1584-byte bulk copy; gw_ipc_alloc
 * buffers are).  The caller orders this against the owners' reads (a barrier
 * over the ranks). */
gw_status gw_moe_ep_dispatch(gw_moe_workspace* workspace, const void* input_bf16, uint32_t rows,
                             const float* inverse_input_scales, const int32_t* dest_rank,
                             const int32_t* dest_row0, void* const* peer_records,
                             uint32_t capacity_rows, void* stream);

/* A small all-to-all exchange that is also a barrier, over peer memory (no collective library call):
 * every rank publishes `count` int32 values (count <= 252; 0 = barrier only) to all ranks and returns,
 * in stream order, once every rank has published its values of the same call -- by which time
 * everything those ranks' GPUs wrote before their call (e.g. records stored into this rank's
 * buffers) is visible here.  gathered[source rank][count] receives the values.
 *   peer_mailboxes  device array of `world` pointers: rank r's mailbox (gw_moe_ep_mailbox_bytes()
 *                   bytes from gw_ipc_alloc, zeroed once before the first call) as mapped here
 *   epoch_counter   one uint32 in this rank's device memory, zeroed once; counts the calls (kept on
 *                   the device so that a replayed step keeps counting); all ranks must make the
 *                   same sequence of calls
 * The wait is bounded (2 s): on a timeout the kernel reports 0x90000000 | source << 8 | rank through
 * gw_debug_kernel_error and returns.  At most 8 ranks, each on its own GPU. */
size_t gw_moe_ep_mailbox_bytes(void);
gw_status gw_moe_ep_exchange(const int32_t* payload, uint32_t count, void* const* peer_mailboxes, uint32_t rank,
                             uint32_t world, uint32_t* epoch_counter, int32_t* gathered, void* stream);

/* The destination tables on the device, without a host round trip: from
 * counts[source rank][expert id] (world x 128 int32, the all-gathered routing
 * histograms) and physical[expert id] (position of the expert in (owner, id)
 * order) compute dest_row0[128] for this rank and its own group boundaries
 * local_offsets[128 / world + 1].  Rows of an expert sit expert-major on the
 * owner, source ranks in rank order.  A record that would fall outside
 * capacity_rows is dropped by the dispatch and reported through the kernel
 * error word. */
gw_status gw_moe_ep_tables(const int32_t* counts, const int32_t* physical, uint32_t rank, uint32_t world,
                           int32_t* dest_row0, int32_t* local_offsets, int32_t* segment_start,
                           int32_t* home_base, void* stream);
/* segment_start / home_base (both NULL, or world x 128/world int32 each, world <= 8)
 * describe the way home for gw_moe_ep_run_experts: rows [segment_start[s][j], ...)
 * of this rank's j-th expert came from rank s, where they are rows home_base[s][j]..
 * of its expert-sorted order. */

/* The same exchange with the down projection at the tokens' home: 14 times fewer bytes come back over
 * NVLink (a 416-byte record of the quantised down input -- 352 B of E2M1, 44 scale bytes in K order,
 * padding -- instead of a 5632-byte BF16 result row), for the price of every rank holding the down
 * matrices of all 128 experts (a third of the expert weights).  The arithmetic per row is unchanged, so
 * the layer's output is the same bits.
 *   gw_moe_ep_run_gate_up      owner side: gate/up GEMM + GeGLU + FP4 quantisation over the records this
 *                              rank received (arguments as gw_moe_ep_run_experts), then one activation
 *                              record per row, in the same expert-major order, into
 *                              `activation_records` (capacity x gw_moe_ep_activation_record_bytes(),
 *                              a gw_ipc_alloc buffer that the peers read)
 *   gw_moe_ep_finish_at_home   home side, after a barrier: fetches the record of each of this rank's
 *                              8 x rows assignments from its owner (same addressing as
 *                              gw_moe_ep_combine) into the routing workspace's own expert-sorted order,
 *                              runs the grouped down GEMM over them with `down_table` (an expert table
 *                              whose 128 entries carry the down projection; gate and up may be
 *                              GW_STORAGE_ABSENT) and folds each token's eight rows in expert order. */
size_t gw_moe_ep_activation_record_bytes(void);
gw_status gw_moe_ep_run_gate_up(gw_moe_workspace* workspace, const void* records, const int32_t* offsets,
                                uint32_t first_expert, uint32_t expert_count, uint32_t total_rows,
                                const gw_expert_table* table, void* activation_records, void* stream);
gw_status gw_moe_ep_finish_at_home(gw_moe_workspace* workspace, uint32_t rows, const int32_t* dest_rank,
                                   const int32_t* dest_row0, void* const* peer_activation_records,
                                   uint32_t capacity_rows, const gw_expert_table* down_table, void* output_bf16,
                                   void* stream);

/* Owner side: grouped gate/up GEMM + GeGLU + grouped down GEMM over the
 * records this rank received, grouped by expert as `offsets` (expert_count + 1
 * entries, on the device) says; `total_rows` is an upper bound known to the host
 * (the true count is offsets[expert_count]), so no read-back is needed; BF16 results [total_rows, 2816] in the same
 * order go to `down_bf16` (a gw_ipc_alloc buffer when peers read it). */
gw_status gw_moe_ep_run_experts(gw_moe_workspace* workspace, const void* records, const int32_t* offsets,
                                uint32_t first_expert, uint32_t expert_count, uint32_t total_rows,
                                const gw_expert_table* table, void* down_bf16,
                                const int32_t* segment_start, const int32_t* home_base,
                                void* const* peer_returned, uint32_t home_capacity_rows, uint32_t world,
                                void* stream);
/* With peer_returned != NULL (one [8 * tokens, 2816] BF16 gw_ipc_alloc buffer per
 * rank, pointers in device memory) the down GEMM's epilogue stores every result row
 * straight into its source rank's buffer, at the row's position in that rank's
 * expert-sorted order, so the transfer home overlaps the GEMM; down_bf16 is then
 * unused and the source folds its rows with gw_moe_combine after a barrier;
 * home_capacity_rows is the row count of each of those buffers (a row whose home
 * would lie outside is not stored and is reported through the kernel error word).
 * With peer_returned == NULL the rows stay in down_bf16 and gw_moe_ep_combine pulls
 * them.
 * Offsets that describe more than total_rows rows are clamped to total_rows and
 * reported through the kernel error word: nothing is read or written beyond the
 * declared capacity. */

/* Ordered BF16 fold (moe.cu:446-456) of each token's eight result rows, read
 * from their owners: row dest_row0[e] + position of peer_down[dest_rank[e]].
 * capacity_rows is the row count of every owner's buffer; a row that would lie
 * outside is not read (it counts as zero) and is reported through the kernel
 * error word. */
gw_status gw_moe_ep_combine(gw_moe_workspace* workspace, uint32_t rows, const int32_t* dest_rank,
                            const int32_t* dest_row0, void* const* peer_down, uint32_t capacity_rows,
                            void* output_bf16, void* stream);

/* Last kernel-reported error word of this process's device (0 = none); set by
 * bounded waits inside the tensor-core kernels.  Synchronises the device. */
uint32_t gw_debug_kernel_error(void);

#ifdef __cplusplus
}
#endif
#endif /* GEWELL_B200_H_ */
