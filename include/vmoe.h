/*
 * vmoe.h -- C ABI of the B200 (sm_100a) fused NVFP4 MoE expert layer.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*), returns an int status (VMOE_OK == 0) and
 * neither allocates nor synchronises; the caller owns every buffer, including the
 * workspace blob whose size vmoe_workspace_bytes() reports.  This is the surface a
 * binding of the reference's operator would call in place of its pybind11
 * extension functions (reference: fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu
 * :574-656 `verdict_cooperative_tma_forward`, :1022-1031 the pybind module; and
 * fused-moe/csrc/verdict_moe_ext.cu:358-433, :578-582 for the scalar pipeline).
 *
 * Tensor layouts are the reference's (fused-moe/verdict_moe.py:571-575, :519-520):
 *   hidden   [M, K]        bf16
 *   w13      [E, 2N, K/2]  u8, two E2M1 codes per byte, even k in the low nibble;
 *                          rows 0..N-1 = gate, N..2N-1 = up
 *   w13_sf   [E, 2N, K/16] u8, E4M3 block scales, linear (not swizzled)
 *   w13_gs   [E]           f32 per-expert global scale (the reference's alpha1)
 *   w2       [E, K, N/2]   u8;  w2_sf [E, K, N/16] u8;  w2_gs [E] f32 (alpha2)
 *   out      [M, K]        bf16
 * K = hidden size, N = expert intermediate size, E = experts held by this GPU,
 * T = experts per token.
 */
#ifndef VMOE_H_
#define VMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VMOE_ABI_VERSION 4

enum vmoe_status {
    VMOE_OK = 0,
    VMOE_ERR_NULL = 1,       /* a required pointer is NULL */
    VMOE_ERR_SHAPE = 2,      /* unsupported K / N / E / T / M */
    VMOE_ERR_ALIGN = 3,      /* a pointer is not 16-byte aligned */
    VMOE_ERR_WORKSPACE = 4,  /* workspace too small */
    VMOE_ERR_CUDA = 5,       /* a CUDA call failed; cudaGetLastError has details */
    VMOE_ERR_TIMEOUT = 6,    /* a bounded device-side wait ran out (read from the status word) */
    VMOE_ERR_SCALE = 7,      /* a block-scale byte has its sign bit set (NVFP4 scales are unsigned) */
    VMOE_ERR_LIMIT = 8,      /* size beyond a stated fixed maximum, or an expert id outside its range */
    VMOE_ERR_PEER = 9        /* expert parallelism: another rank reported a failure for this call */
};

/* Problem shape.  Replaces the reference's compile-time HIDDEN = 4096 and the
 * (K, N_half, num_pairs) integer arguments of its forward functions
 * (fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:32, :594-596). */
typedef struct vmoe_shape {
    int32_t hidden;       /* K: multiple of 128 (tensor-core path: multiple of 256; streaming GEMV path: <= 4096) */
    int32_t inter;        /* N: multiple of 128 (tensor-core path: multiple of 256; streaming GEMV path: <= 1024) */
    int32_t num_experts;  /* E: routed experts whose weights this GPU holds */
    int32_t topk;         /* T: 1..16 */
    int32_t max_tokens;   /* largest M the workspace must serve */
    int32_t has_shared;   /* 1: an always-on shared expert is applied to every token */
    int32_t num_global_experts; /* width of router logits / range of topk ids (== E without expert parallelism) */
    int32_t path;         /* 0 = automatic (tensor-core path when the weights carry prepared scales, else the
                             streaming GEMV path), 1 = streaming GEMV on CUDA cores, 2 = tcgen05 tensor-core path */
} vmoe_shape;

enum vmoe_path { VMOE_PATH_AUTO = 0, VMOE_PATH_GEMV = 1, VMOE_PATH_TC = 2 };

/* One set of NVFP4 expert weights (device pointers).  Replaces the (w1, w1_sf,
 * w1_alpha, w2, w2_sf, w2_alpha) tensor arguments of the reference's forward
 * (…tma_ext.cu:575-581); the per-pair alpha gather of fused-moe/verdict_moe.py
 * :499-513 happens on the device from the per-expert arrays. */
typedef struct vmoe_weights {
    const uint8_t* w13;
    const uint8_t* w13_sf;
    const float*   w13_gs;
    const uint8_t* w2;
    const uint8_t* w2_sf;
    const float*   w2_gs;
    /* Optional: the same block scales re-laid by vmoe_prepare_sf for the tensor-core path
     * ([rows/128][K/64][512 bytes]); NULL = not prepared.  The reference has no such copy: it
     * explicitly keeps scales linear (fused-moe/FINAL_SUMMARY.md:104-111). */
    const uint8_t* w13_sf_atoms;
    const uint8_t* w2_sf_atoms;
} vmoe_weights;

/* Byte offsets of the intermediate tables inside the workspace, so that a test or
 * a profiler can read each stage.  Mirrors the scratch tensors the reference
 * preallocates in fused-moe/verdict_moe.py:243-414 (input_fp4/input_sf,
 * inter_fp4/inter_sf, pair_output_f32, expert id / weight / token tables). */
typedef struct vmoe_ws_layout {
    size_t total_bytes;
    size_t topk_ids;        /* int32 [M, T] */
    size_t topk_weights;    /* f32   [M, T] */
    size_t expert_offsets;  /* int32 [E + 2]: exclusive scan of pairs per expert; entry E.. = shared expert */
    size_t sorted_pair;     /* int32 [P + M]: flat pair index of each sorted slot */
    size_t pair_slot;       /* int32 [P]: sorted slot of each pair, -1 when its expert is not local */
    size_t gather_idx;      /* int32 [P + M]: source token of each sorted slot */
    size_t scatter_weights; /* f32   [P + M]: router weight of each sorted slot (1.0 for the shared expert) */
    size_t units;           /* int32 [max_units, 4]: (expert, first slot, tokens, 0) work units of the GEMV path */
    size_t counters;        /* int32 [8]: 0 = number of units, 1 = number of slots, 2..3 = work queues, 4 = status word */
    size_t act_q;           /* u8 [M, K/2] quantised activations */
    size_t act_sf;          /* u8 [M, K/16] */
    size_t inter_q;         /* u8 [P + M, N/2] quantised SwiGLU output per sorted slot */
    size_t inter_sf;        /* u8 [P + M, N/16] */
    size_t pair_out;        /* f32 [P + M, K] weighted down-projection rows per sorted slot */
    size_t bitmap;          /* u32 [E, ceil(M/32)] scratch of the permutation */
    size_t word_prefix;     /* int32 [E, ceil(M/32)] scratch of the permutation */
    size_t tc_units;        /* int32 [max_tc_units, 4]: (expert, first slot, tokens, UMMA N) units of <= 16 tokens
                               (weights-as-rows kernel) or <= 128 tokens (token-major kernel) */
    size_t tc_unit_base;    /* int32 [E + 1]: first tensor-core unit of each expert */
    size_t act_q_sorted;    /* u8 [P + M, K/2] quantised activations in sorted-slot order (B operand of GEMM1) */
    size_t act_sf_atoms;    /* u8 [max_tc_units, K/64, 512] activation scales, 128-row x 4-scale atoms per unit */
    size_t inter_sf_atoms;  /* u8 [max_tc_units, N/64, 512] intermediate scales, same layout */
    size_t unit_done;       /* int32 [max_tc_units]: gate_up row tiles finished per unit (the down projection of a unit
                               starts when all of them are) */
    size_t token_done;      /* int32 [small-batch tokens, K/128]: down-projection rows finished per token and column tile */
    size_t token_expect;    /* int32 [small-batch tokens]: rows a token receives (its local pairs + the shared expert) */
} vmoe_ws_layout;

int         vmoe_abi_version(void);
const char* vmoe_status_string(int status);

/* Workspace sizing.  Replaces VerdictMoEExperts.setup_buffers / workspace_shapes
 * (fused-moe/verdict_moe.py:224-238, :243-414). */
size_t vmoe_workspace_bytes(const vmoe_shape* shape);
int    vmoe_workspace_layout(const vmoe_shape* shape, vmoe_ws_layout* out);

/* Router: fp32 softmax over all experts, top-T by probability (lowest expert id
 * wins ties, descending order), renormalised.  Replaces moe_topk_select
 * (fused-moe/csrc/megakernel_v1.cu:491-537).  logits [M, E] f32. */
int vmoe_route(const float* logits, int32_t M, int32_t E, int32_t T,
               int32_t* topk_ids, float* topk_weights, void* stream);

/* Permutation by expert: stable sort of the M*T pairs by (local) expert id,
 * expert offsets, gather / scatter tables and the GEMV work-unit list, written into
 * the workspace at the offsets of vmoe_workspace_layout().  Replaces
 * build_group_tables (fused-moe/csrc/verdict_fused_grouped.cu:655-691) and the flat
 * pair tables + expert_map remap of fused-moe/verdict_moe.py:473-477, :490-496.
 * expert_map [num_global_experts] int32 (-1 = not local) or NULL. */
int vmoe_build_tables(const vmoe_shape* shape, const int32_t* topk_ids,
                      const float* topk_weights, const int32_t* expert_map,
                      int32_t M, void* workspace, size_t workspace_bytes, void* stream);

/* Activation quantiser bf16 -> NVFP4 (per-16 E4M3 block scale, no global scale).
 * Replaces the prologue of the fused kernel (…tma_ext.cu:249-279) and
 * bf16_to_nvfp4_e4m3_kernel (fused-moe/csrc/verdict_fused_ext.cu:154-192). */
int vmoe_quantize(const void* x_bf16, int32_t rows, int32_t K,
                  uint8_t* packed, uint8_t* sf, void* stream);

/* One-time re-layout of linear E4M3 block scales [rows, K/16] into the 128-row x 4-scale atoms the
 * tcgen05 block-scaled MMA reads ([rows/128][K/64][512 bytes], same size as the input); rows must
 * be a multiple of 128, K of 64.  NaN patterns are stored as 0x00 (they decode to zero in the
 * reference, …tma_ext.cu:48-55); *bad_count (device int32, caller zeroes it) is incremented for
 * every byte with the sign bit set -- such weights must not be used with the tensor-core path.
 * Done once per weight tensor at load time; the reference has no counterpart (its scales stay
 * linear, fused-moe/verdict_moe.py:519-520). */
int vmoe_prepare_sf(const uint8_t* sf, int64_t rows, int32_t K, uint8_t* atoms,
                    int32_t* bad_count, void* stream);

/* Decode NVFP4 to f32: value = e2m1(code) * e4m3(block scale) * global_scale[row_group].
 * rows_per_scale rows share one entry of global_scale (NULL = 1.0).  Replaces
 * read_nvfp4 / decode_fp4 / decode_e4m3fn (fused-moe/csrc/verdict_moe_ext.cu:86-116). */
int vmoe_dequantize(const uint8_t* packed, const uint8_t* sf, const float* global_scale,
                    int64_t rows, int32_t K, int64_t rows_per_scale, float* out, void* stream);

/* The fused layer.  Replaces verdict_cooperative_tma_forward (…tma_ext.cu:574-656)
 * plus the host glue of VerdictMoEExperts.apply (fused-moe/verdict_moe.py:421-553).
 * Give either router logits [M, num_global_experts] f32 (routing runs on the
 * device) or topk_ids / topk_weights [M, T] (pre-routed, the reference's slot);
 * shared may be NULL when shape->has_shared == 0. */
int vmoe_forward(const vmoe_shape* shape, const vmoe_weights* routed,
                 const vmoe_weights* shared, const void* hidden_bf16,
                 const float* router_logits, const int32_t* topk_ids,
                 const float* topk_weights, const int32_t* expert_map,
                 void* out_bf16, int32_t M, void* workspace, size_t workspace_bytes,
                 void* stream);

/* Optional neighbours of the layer, fused around it (all pointers may be NULL = not used). */
typedef struct vmoe_extras {
    const void* gate_weight;     /* router matrix [num_global_experts, hidden]; logits = hidden @ gate_weight^T in
                                    f32 on the device, then routed.  Used when router_logits, topk_ids are NULL.
                                    Replaces moe_gate_distributed (fused-moe/csrc/megakernel_v1.cu:455-489). */
    int32_t     gate_dtype;      /* 0 = f32 (the reference's type), 1 = bf16 */
    const void* residual_bf16;   /* [M, hidden]: out = bf16(residual + bf16(layer output)), the residual add the
                                    reference's whole-model kernel performs after the MoE block
                                    (fused-moe/csrc/megakernel_v1.cu:1431-1505); may alias out_bf16 */
    /* RMSNorm + NVFP4 activation quantisation of the NEXT layer's input, fused behind the combine (+ residual):
     * y = bf16(out * rsqrt(mean(out^2) + eps) * gamma), then y quantised per 16 elements exactly as vmoe_quantize
     * does.  Replaces rmsnorm_parallel + rmsnorm_apply_and_quantize (fused-moe/csrc/megakernel_v1.cu:257-352).
     * next_norm_weight == NULL: not used. */
    const float* next_norm_weight;  /* [hidden] f32 gamma */
    float        next_norm_eps;
    void*        next_normed_bf16;  /* out [M, hidden] bf16 normalised rows (the next router's input); may be NULL */
    uint8_t*     next_act_q;        /* out [M, hidden/2] E2M1 codes */
    uint8_t*     next_act_sf;       /* out [M, hidden/16] E4M3 block scales */
    /* This layer's input already quantised (the next_act_q / next_act_sf a previous layer wrote): the activation
     * quantiser is skipped and these codes are used as they are.  hidden_bf16 is then only read by the router
     * projection (gate_weight) and may be NULL without one. */
    const uint8_t* hidden_q;
    const uint8_t* hidden_sf;
} vmoe_extras;

/* vmoe_forward with the optional neighbours above.  extras == NULL behaves exactly like vmoe_forward. */
int vmoe_forward_ex(const vmoe_shape* shape, const vmoe_weights* routed,
                    const vmoe_weights* shared, const void* hidden_bf16,
                    const float* router_logits, const int32_t* topk_ids,
                    const float* topk_weights, const int32_t* expert_map,
                    void* out_bf16, int32_t M, void* workspace, size_t workspace_bytes,
                    const vmoe_extras* extras, void* stream);

/* RMSNorm + activation quantisation alone, over rows x [rows, K] bf16 (the arithmetic of vmoe_extras.next_norm_*;
 * the first layer of a stack needs it once).  y_bf16 may be NULL.  K a multiple of 16.  Replaces
 * rmsnorm_parallel + rmsnorm_apply_and_quantize (fused-moe/csrc/megakernel_v1.cu:257-352). */
int vmoe_rmsnorm_quantize(const void* x_bf16, const float* gamma, float eps, int32_t rows, int32_t K,
                          void* y_bf16, uint8_t* packed, uint8_t* sf, void* stream);

/* Router projection alone: logits[M, E] (f32) = hidden[M, K] (bf16) @ gate_weight[E, K]^T, f32 accumulation in a
 * fixed order (deterministic).  K a multiple of 256.  Replaces moe_gate_distributed
 * (fused-moe/csrc/megakernel_v1.cu:455-489). */
int vmoe_router_gemv(const void* hidden_bf16, const void* gate_weight, int32_t gate_dtype,
                     int32_t M, int32_t K, int32_t E, float* logits, void* stream);

/* Individual stages of vmoe_forward over an already built workspace (tables and
 * quantised activations present).  For stage-wise parity checks and per-kernel
 * timing, as the reference's per_kernel_timing (fused-moe/csrc/verdict_moe_ext.cu
 * :482-573). */
int vmoe_stage_gate_up(const vmoe_shape* shape, const vmoe_weights* routed,
                       const vmoe_weights* shared, int32_t M, void* workspace, void* stream);
int vmoe_stage_down(const vmoe_shape* shape, const vmoe_weights* routed,
                    const vmoe_weights* shared, int32_t M, void* workspace, void* stream);
int vmoe_stage_combine(const vmoe_shape* shape, int32_t M, void* workspace,
                       void* out_bf16, void* stream);
/* gate_up and down projection as the forward runs them on the tensor-core path -- one launch of the fused kernel for
 * small batches, the two token-major kernels for large ones -- without quantiser and combine: the dominant kernel(s)
 * alone, for the roofline figure.  VMOE_ERR_SHAPE on the streaming GEMV path. */
int vmoe_stage_experts(const vmoe_shape* shape, const vmoe_weights* routed,
                       const vmoe_weights* shared, int32_t M, void* workspace, void* stream);

/* Reads (and clears) the device status word of a workspace after the caller has
 * synchronised the stream: VMOE_OK or VMOE_ERR_TIMEOUT.  The reference has no
 * counterpart (its waits are unbounded: …tma_ext.cu:156-167). */
int vmoe_read_status(void* workspace, const vmoe_shape* shape, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Expert parallelism across the GPUs of one NVLink box.  One process per GPU.  Every rank owns
 * `experts_per_rank` consecutive experts (gpu = e / experts_per_rank, as
 * fused-moe/p2p_moe_routing.py:26-33) and a "slab" of device memory that its peers write into:
 * quantised token rows + (local expert, pair, weight) records on the way in, weighted fp32 output
 * rows on the way back.  The reference only sketches this exchange
 * (fused-moe/p2p_moe_routing.py:113-131; its working variants replicate all tokens and all-reduce,
 * fused-moe/patches/p2p_ep_communicator.py:99-155).
 * Set-up (once, outside the forward path): vmoe_ep_alloc a slab of vmoe_ep_slab_bytes, export its
 * IPC handle, exchange the 64-byte handles between ranks by any means, vmoe_ep_ipc_open the
 * peers' handles and fill vmoe_ep_ctx.slab[] (own entry = own pointer). */
typedef struct vmoe_ep_ctx {
    int32_t rank, world;          /* world <= 16 */
    int32_t experts_per_rank;
    int32_t capacity;             /* rows one source rank may send to one destination rank per call */
    int32_t max_local_tokens;     /* tokens a rank may bring to one call */
    int32_t wait_limit_us;        /* limit of every cross-GPU wait in microseconds; 0 = one second */
    int32_t reserved[2];
    void*   slab[16];             /* slab of every rank as mapped into this process */
} vmoe_ep_ctx;

size_t vmoe_ep_slab_bytes(const vmoe_ep_ctx* ctx, const vmoe_shape* shape);
size_t vmoe_ep_workspace_bytes(const vmoe_ep_ctx* ctx, const vmoe_shape* shape);
int    vmoe_ep_alloc(size_t bytes, void** out);          /* cudaMalloc + clear; set-up only */
int    vmoe_ep_free(void* slab);
int    vmoe_ep_ipc_export(void* slab, void* handle_out_64_bytes);
int    vmoe_ep_ipc_open(const void* handle_64_bytes, void** out);
int    vmoe_ep_ipc_close(void* mapped);

/* One expert-parallel forward on this rank: route the M local tokens, dispatch them to the ranks
 * that own their experts, run the local experts on the rows that arrived (tensor-core path; weights
 * must carry prepared scales), send each weighted row back to its owner, reduce (+ residual_bf16
 * [M, hidden] when not NULL, as vmoe_extras.residual_bf16; may alias out_bf16).  shape->num_experts =
 * experts_per_rank, shape->num_global_experts = world * experts_per_rank.  Every rank must make the
 * same sequence of calls: the call number is kept in device memory inside the workspace (zeroed by the
 * caller once, before the first call, together with the slab) and advanced by the call itself, so a
 * call has no per-call host state and may be captured in a CUDA graph and replayed.
 * Every cross-GPU wait is bounded (ctx->wait_limit_us).  Status word after the call: VMOE_ERR_TIMEOUT
 * = a wait ran out on this rank; VMOE_ERR_LIMIT = this rank sent more than `capacity` rows to one
 * destination; VMOE_ERR_PEER = another rank reported one of the two.  In all three cases the output
 * of this call is not written on any rank that saw the mark; the status word stays set (and marks
 * this rank's later calls) until vmoe_ep_read_status has read it. */
int vmoe_ep_forward(const vmoe_ep_ctx* ctx, const vmoe_shape* shape, const vmoe_weights* routed,
                    const vmoe_weights* shared, const void* hidden_bf16, const float* router_logits,
                    const void* residual_bf16, void* out_bf16, int32_t M, void* workspace,
                    size_t workspace_bytes, void* stream);
/* Status word of an expert-parallel workspace (synchronises the stream, clears the word). */
int vmoe_ep_read_status(const vmoe_ep_ctx* ctx, const vmoe_shape* shape, void* workspace, void* stream);

/* Permutation by expert for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.  Same tables as vmoe_build_tables, but written to arrays the
 * caller passes (expert_offsets [E + 2], sorted_pair / gather_idx / scatter_weights
 * [M*T + (has_shared ? M : 0)], pair_slot [M*T]) and with all scratch in a fixed array inside the
 * library, so the call needs no workspace and performs no allocation of any kind.  It is meant
 * for hosts that only own the buffers they were given at this point -- a serving worker whose
 * memory pool already fills the GPU, or a thin FFI binding with no allocator.
 * Limits: M <= 1024 tokens, E <= 1024 local experts, T <= 16 (VMOE_ERR_LIMIT beyond them); the
 * scratch array is about 342 KiB per GPU that loads the library and is kept until the process
 * exits.  The first call on each device looks up the array's device address (that device must
 * be current); make that first call before any stream capture.  All calls share the one array,
 * which is cleared at the start of each call: calls that overlap on the GPU (two streams, two
 * threads) race and must be serialised by the caller.  The looked-up address is kept for the
 * life of the process: do not use the entry point across a cudaDeviceReset.  With an expert_map
 * every id must lie in [0, length of expert_map) -- the length is not an argument, so ids cannot
 * be range-checked here (negative ids are dropped); without one, ids outside [0, E) are dropped. */
int vmoe_permute_noalloc(const int32_t* topk_ids, const float* topk_weights,
                         const int32_t* expert_map, int32_t M, int32_t T, int32_t E,
                         int32_t has_shared, int32_t* expert_offsets, int32_t* sorted_pair,
                         int32_t* pair_slot, int32_t* gather_idx, float* scatter_weights,
                         void* stream);

#ifdef __cplusplus
}
#endif
#endif /* VMOE_H_ */
