// C ABI: argument validation, workspace layout, stage sequencing.  No allocation, no
// synchronisation; every launch goes to the caller's stream.
#include "vmoe_common.cuh"

#include <string.h>

#ifdef VMOE_TIMELINE
namespace vmoe { unsigned long long* g_vmoe_timeline = nullptr; }
// development builds only: 32 x u64 device buffer that the small-batch kernels write %globaltimer marks into
extern "C" int vmoe_debug_set_timeline(void* device_buffer) { vmoe::g_vmoe_timeline = static_cast<unsigned long long*>(device_buffer); return 0; }
#endif

namespace vmoe {

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int max_units(const vmoe_shape* s) {
    const long long P = (long long)s->max_tokens * s->topk + (s->has_shared ? s->max_tokens : 0);
    return (int)(s->num_experts + 1 + (P + TOK_PER_UNIT - 1) / TOK_PER_UNIT);
}

// Units carry at most 16 tokens while the batch averages <= 10 pairs per expert (weights-as-rows kernel: gate_up
// and down in one launch, a small token tile leaves shared memory for a deep weight ring; experts above 16 tokens
// are split and re-read through L2) and 128 tokens above (token-major kernels).  The crossover was measured on the
// 512-expert top-10 layer: 384 tokens (7.5 pairs per expert) 625 against 658 us, 512 tokens equal, 640 tokens
// (12.5 per expert) 700 against 667 us.  VMOE_SMALL_PER_EXPERT overrides it (up to the 16 the workspace is sized for).
constexpr long long TC_SMALL_PER_EXPERT = 10;         // default crossover (pairs per expert), measured
constexpr long long TC_SMALL_PER_EXPERT_MAX = 16;     // what the workspace is sized for
int tc_unit_cap(const vmoe_shape& s, int M) {
    const long long pairs = (long long)M * s.topk;
    long long per = tuning("VMOE_SMALL_PER_EXPERT", (int)TC_SMALL_PER_EXPERT);
    if (per > TC_SMALL_PER_EXPERT_MAX) per = TC_SMALL_PER_EXPERT_MAX;
    return pairs <= per * s.num_experts ? TC_UNIT_TOK_SMALL : TC_UNIT_TOK_PREFILL;
}

// Largest batch that can take the weights-as-rows kernel (and with it the in-kernel combine).
int small_batch_tokens(const vmoe_shape* s) {
    const long long m = TC_SMALL_PER_EXPERT_MAX * s->num_experts / s->topk;
    return (int)(m < s->max_tokens ? m : s->max_tokens);
}

// Entries of the tensor-core unit list: every expert (+ shared) may end with one partial unit; full units are 16
// tokens in the small regime (which ends at 7 E pairs + their shared rows) and 128 tokens above it.
int max_tc_units(const vmoe_shape* s) {
    const long long S = (long long)s->max_tokens * s->topk + (s->has_shared ? s->max_tokens : 0);
    long long small_slots = (long long)small_batch_tokens(s) * (s->topk + (s->has_shared ? 1 : 0));
    if (small_slots > S) small_slots = S;
    const long long a = (S + TC_UNIT_TOK_PREFILL - 1) / TC_UNIT_TOK_PREFILL, b = (small_slots + TC_UNIT_TOK_SMALL - 1) / TC_UNIT_TOK_SMALL;
    return (int)(s->num_experts + 2 + (a > b ? a : b));
}

// The streaming GEMV kernels keep one activation row per 128 consumer threads x 32 elements.
static bool gemv_shape_ok(const vmoe_shape* s) { return s->hidden <= 4096 && s->inter <= 1024; }

static int check_shape(const vmoe_shape* s) {
    if (!s) return VMOE_ERR_NULL;
    if (s->hidden <= 0 || s->hidden % 128 || s->hidden > (1 << 20)) return VMOE_ERR_SHAPE;
    if (s->inter <= 0 || s->inter % 128 || s->inter > (1 << 20)) return VMOE_ERR_SHAPE;
    if (s->num_experts <= 0 || s->topk <= 0 || s->topk > MAX_TOPK) return VMOE_ERR_SHAPE;
    if (s->max_tokens < 0) return VMOE_ERR_SHAPE;
    if (s->num_global_experts < s->num_experts) return VMOE_ERR_SHAPE;
    if (s->topk > s->num_global_experts) return VMOE_ERR_SHAPE;
    if (s->path < 0 || s->path > 2) return VMOE_ERR_SHAPE;
    if (s->path == VMOE_PATH_TC && (s->hidden % 256 || s->inter % 256)) return VMOE_ERR_SHAPE;
    if (s->path == VMOE_PATH_GEMV && !gemv_shape_ok(s)) return VMOE_ERR_SHAPE;
    return VMOE_OK;
}

int compute_layout(const vmoe_shape* s, vmoe_ws_layout* L, int tc_units_override) {
    const int rc = check_shape(s);
    if (rc) return rc;
    const size_t M = (size_t)s->max_tokens, T = s->topk, E = s->num_experts, K = s->hidden, N = s->inter;
    const size_t P = M * T, S = P + M;          // S: sorted slots incl. shared expert rows
    const size_t words = (M + 31) / 32;
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o = off; off = align_up(off + bytes, 256); return o; };
    memset(L, 0, sizeof(*L));
    L->counters        = take(CNT_N * 4);
    L->topk_ids        = take(P * 4);
    L->topk_weights    = take(P * 4);
    L->expert_offsets  = take((E + 2) * 4);
    L->sorted_pair     = take(S * 4);
    L->pair_slot       = take(P * 4);
    L->gather_idx      = take(S * 4);
    L->scatter_weights = take(S * 4);
    L->units           = take((size_t)max_units(s) * 16);
    L->act_q           = take(M * K / 2);
    L->act_sf          = take(M * K / 16);
    L->inter_q         = take(S * N / 2);
    L->inter_sf        = take(S * N / 16);
    L->pair_out        = take(S * K * 4);
    L->bitmap          = take(E * words * 4);
    L->word_prefix     = take(E * words * 4);
    const size_t TU = tc_units_override > 0 ? (size_t)tc_units_override : (size_t)max_tc_units(s);
    L->tc_units        = take(TU * 16);
    L->tc_unit_base    = take((E + 1) * 4);
    L->act_q_sorted    = take(S * K / 2);
    L->act_sf_atoms    = take(TU * (K / 64) * 512);
    L->inter_sf_atoms  = take(TU * ((N + 63) / 64) * 512);
    const size_t small = (size_t)small_batch_tokens(s);
    L->unit_done       = take(TU * 4);
    L->token_done      = take(small * (K / TC_TILE_ROWS) * 4);
    L->token_expect    = take(small * 4);
    L->total_bytes     = off;
    return VMOE_OK;
}

int resolve_workspace(const vmoe_shape* s, void* base, Workspace* ws, int tc_units_override) {
    vmoe_ws_layout L;
    const int rc = compute_layout(s, &L, tc_units_override);
    if (rc) return rc;
    uint8_t* b = static_cast<uint8_t*>(base);
    ws->counters        = reinterpret_cast<int32_t*>(b + L.counters);
    ws->topk_ids        = reinterpret_cast<int32_t*>(b + L.topk_ids);
    ws->topk_weights    = reinterpret_cast<float*>(b + L.topk_weights);
    ws->expert_offsets  = reinterpret_cast<int32_t*>(b + L.expert_offsets);
    ws->sorted_pair     = reinterpret_cast<int32_t*>(b + L.sorted_pair);
    ws->pair_slot       = reinterpret_cast<int32_t*>(b + L.pair_slot);
    ws->gather_idx      = reinterpret_cast<int32_t*>(b + L.gather_idx);
    ws->scatter_weights = reinterpret_cast<float*>(b + L.scatter_weights);
    ws->units           = reinterpret_cast<int4*>(b + L.units);
    ws->act_q           = b + L.act_q;
    ws->act_sf          = b + L.act_sf;
    ws->inter_q         = b + L.inter_q;
    ws->inter_sf        = b + L.inter_sf;
    ws->pair_out        = reinterpret_cast<float*>(b + L.pair_out);
    ws->bitmap          = reinterpret_cast<uint32_t*>(b + L.bitmap);
    ws->word_prefix     = reinterpret_cast<int32_t*>(b + L.word_prefix);
    ws->tc_units        = reinterpret_cast<int4*>(b + L.tc_units);
    ws->tc_unit_base    = reinterpret_cast<int32_t*>(b + L.tc_unit_base);
    ws->act_q_sorted    = b + L.act_q_sorted;
    ws->act_sf_atoms    = b + L.act_sf_atoms;
    ws->inter_sf_atoms  = b + L.inter_sf_atoms;
    ws->row_dst         = nullptr;
    ws->unit_done       = reinterpret_cast<int32_t*>(b + L.unit_done);
    ws->token_done      = reinterpret_cast<int32_t*>(b + L.token_done);
    ws->token_expect    = reinterpret_cast<int32_t*>(b + L.token_expect);
    ws->tc_unit_capacity = tc_units_override > 0 ? tc_units_override : max_tc_units(s);
    ws->small_tokens    = small_batch_tokens(s);
    ws->pair_rows_bf16  = 0;
#ifdef VMOE_TIMELINE
    ws->timeline        = g_vmoe_timeline;
#else
    ws->timeline        = nullptr;
#endif
    return VMOE_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static int check_weights(const vmoe_weights* w) {
    if (!w || !w->w13 || !w->w13_sf || !w->w13_gs || !w->w2 || !w->w2_sf || !w->w2_gs) return VMOE_ERR_NULL;
    if (!aligned16(w->w13) || !aligned16(w->w13_sf) || !aligned16(w->w2) || !aligned16(w->w2_sf)) return VMOE_ERR_ALIGN;
    return VMOE_OK;
}

static WeightSet to_set(const vmoe_weights* w) {
    WeightSet s{};
    if (w) { s.w13 = w->w13; s.w13_sf = w->w13_sf; s.w13_gs = w->w13_gs; s.w2 = w->w2; s.w2_sf = w->w2_sf; s.w2_gs = w->w2_gs; }
    return s;
}

static PreparedSet to_prep(const vmoe_weights* r, const vmoe_weights* sh) {
    PreparedSet p{};
    if (r) { p.w13_sf_atoms = r->w13_sf_atoms; p.w2_sf_atoms = r->w2_sf_atoms; }
    if (sh) { p.shared_w13_sf_atoms = sh->w13_sf_atoms; p.shared_w2_sf_atoms = sh->w2_sf_atoms; }
    return p;
}

// which path a call takes; VMOE_ERR_* (negative of nothing: plain status) when the request cannot be met
static int pick_path(const vmoe_shape* s, const vmoe_weights* routed, const vmoe_weights* shared, int* path) {
    const bool prepared = routed->w13_sf_atoms && routed->w2_sf_atoms &&
                          (!s->has_shared || (shared->w13_sf_atoms && shared->w2_sf_atoms));
    const bool shape_ok = (s->hidden % 256 == 0) && (s->inter % 256 == 0);
    if (s->path == VMOE_PATH_TC) {
        if (!prepared) return VMOE_ERR_NULL;
        if (!shape_ok) return VMOE_ERR_SHAPE;
        *path = VMOE_PATH_TC;
    } else if (s->path == VMOE_PATH_GEMV) {
        *path = VMOE_PATH_GEMV;
    } else {
        *path = (prepared && shape_ok) ? VMOE_PATH_TC : VMOE_PATH_GEMV;
    }
    if (*path == VMOE_PATH_GEMV && !gemv_shape_ok(s)) return VMOE_ERR_SHAPE;
    return VMOE_OK;
}

static int check_call(const vmoe_shape* s, const vmoe_weights* routed, const vmoe_weights* shared, int M,
                      void* workspace) {
    int rc = check_shape(s);
    if (rc) return rc;
    if (M < 0 || M > s->max_tokens) return VMOE_ERR_SHAPE;
    if (!workspace) return VMOE_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return VMOE_ERR_ALIGN;
    if ((rc = check_weights(routed))) return rc;
    if (s->has_shared && (rc = check_weights(shared))) return rc;
    return VMOE_OK;
}

}  // namespace vmoe

using namespace vmoe;

extern "C" {

int vmoe_abi_version(void) { return VMOE_ABI_VERSION; }

const char* vmoe_status_string(int status) {
    switch (status) {
        case VMOE_OK: return "ok";
        case VMOE_ERR_NULL: return "a required pointer is NULL";
        case VMOE_ERR_SHAPE: return "unsupported shape";
        case VMOE_ERR_ALIGN: return "pointer not sufficiently aligned";
        case VMOE_ERR_WORKSPACE: return "workspace too small";
        case VMOE_ERR_CUDA: return "CUDA error";
        case VMOE_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case VMOE_ERR_SCALE: return "block-scale byte with the sign bit set";
        case VMOE_ERR_LIMIT: return "size beyond a fixed maximum, or expert id out of range";
        case VMOE_ERR_PEER: return "another rank reported a failure for this call";
        default: return "unknown status";
    }
}

size_t vmoe_workspace_bytes(const vmoe_shape* shape) {
    vmoe_ws_layout L;
    return compute_layout(shape, &L) == VMOE_OK ? L.total_bytes : 0;
}

int vmoe_workspace_layout(const vmoe_shape* shape, vmoe_ws_layout* out) {
    if (!out) return VMOE_ERR_NULL;
    return compute_layout(shape, out);
}

int vmoe_route(const float* logits, int32_t M, int32_t E, int32_t T, int32_t* topk_ids,
               float* topk_weights, void* stream) {
    if (!logits || !topk_ids || !topk_weights) return VMOE_ERR_NULL;
    if (M < 0 || E <= 0 || T <= 0 || T > MAX_TOPK || T > E) return VMOE_ERR_SHAPE;
    return launch_route(logits, M, E, T, topk_ids, topk_weights, static_cast<cudaStream_t>(stream));
}

int vmoe_build_tables(const vmoe_shape* shape, const int32_t* topk_ids, const float* topk_weights,
                      const int32_t* expert_map, int32_t M, void* workspace, size_t workspace_bytes,
                      void* stream) {
    int rc = check_shape(shape);
    if (rc) return rc;
    if (!topk_ids || !topk_weights || !workspace) return VMOE_ERR_NULL;
    if (M < 0 || M > shape->max_tokens) return VMOE_ERR_SHAPE;
    if (workspace_bytes < vmoe_workspace_bytes(shape)) return VMOE_ERR_WORKSPACE;
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    return launch_tables(*shape, topk_ids, topk_weights, expert_map, M, ws, static_cast<cudaStream_t>(stream),
                         tc_unit_cap(*shape, M));
}

int vmoe_quantize(const void* x_bf16, int32_t rows, int32_t K, uint8_t* packed, uint8_t* sf, void* stream) {
    if (!x_bf16 || !packed || !sf) return VMOE_ERR_NULL;
    if (rows < 0 || K <= 0 || K % SF_BLOCK) return VMOE_ERR_SHAPE;
    if (!aligned16(x_bf16) || (reinterpret_cast<uintptr_t>(packed) & 7)) return VMOE_ERR_ALIGN;
    return launch_quantize(static_cast<const __nv_bfloat16*>(x_bf16), rows, K, packed, sf,
                           static_cast<cudaStream_t>(stream));
}

int vmoe_prepare_sf(const uint8_t* sf, int64_t rows, int32_t K, uint8_t* atoms, int32_t* bad_count, void* stream) {
    if (!sf || !atoms || !bad_count) return VMOE_ERR_NULL;
    if (rows < 0 || rows % 128 || K <= 0 || K % 64) return VMOE_ERR_SHAPE;
    return launch_prep_sf(sf, rows, K, atoms, bad_count, static_cast<cudaStream_t>(stream));
}

int vmoe_dequantize(const uint8_t* packed, const uint8_t* sf, const float* global_scale, int64_t rows,
                    int32_t K, int64_t rows_per_scale, float* out, void* stream) {
    if (!packed || !sf || !out) return VMOE_ERR_NULL;
    if (rows < 0 || K <= 0 || K % SF_BLOCK) return VMOE_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(packed) & 7) return VMOE_ERR_ALIGN;
    return launch_dequantize(packed, sf, global_scale, rows, K, rows_per_scale, out,
                             static_cast<cudaStream_t>(stream));
}

int vmoe_stage_gate_up(const vmoe_shape* shape, const vmoe_weights* routed, const vmoe_weights* shared,
                       int32_t M, void* workspace, void* stream) {
    int rc = check_call(shape, routed, shared, M, workspace);
    if (rc) return rc;
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    int path;
    if ((rc = pick_path(shape, routed, shared, &path))) return rc;
    const WeightSet r = to_set(routed), sh = to_set(shape->has_shared ? shared : nullptr);
    if (path == VMOE_PATH_TC)
        return launch_tc(*shape, r, sh, to_prep(routed, shape->has_shared ? shared : nullptr), M, ws,
                         static_cast<cudaStream_t>(stream), TC_PHASE_GATE_UP);
    return launch_gate_up(*shape, r, sh, M, ws, static_cast<cudaStream_t>(stream));
}

int vmoe_stage_down(const vmoe_shape* shape, const vmoe_weights* routed, const vmoe_weights* shared,
                    int32_t M, void* workspace, void* stream) {
    int rc = check_call(shape, routed, shared, M, workspace);
    if (rc) return rc;
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    int path;
    if ((rc = pick_path(shape, routed, shared, &path))) return rc;
    const WeightSet r = to_set(routed), sh = to_set(shape->has_shared ? shared : nullptr);
    if (path == VMOE_PATH_TC)
        return launch_tc(*shape, r, sh, to_prep(routed, shape->has_shared ? shared : nullptr), M, ws,
                         static_cast<cudaStream_t>(stream), TC_PHASE_DOWN);
    return launch_down(*shape, r, sh, M, ws, static_cast<cudaStream_t>(stream));
}

int vmoe_stage_experts(const vmoe_shape* shape, const vmoe_weights* routed, const vmoe_weights* shared,
                       int32_t M, void* workspace, void* stream) {
    int rc = check_call(shape, routed, shared, M, workspace);
    if (rc) return rc;
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    int path;
    if ((rc = pick_path(shape, routed, shared, &path))) return rc;
    if (path != VMOE_PATH_TC) return VMOE_ERR_SHAPE;
    const WeightSet r = to_set(routed), sh = to_set(shape->has_shared ? shared : nullptr);
    return launch_tc(*shape, r, sh, to_prep(routed, shape->has_shared ? shared : nullptr), M, ws,
                     static_cast<cudaStream_t>(stream), TC_PHASE_GATE_UP | TC_PHASE_DOWN);
}

int vmoe_stage_combine(const vmoe_shape* shape, int32_t M, void* workspace, void* out_bf16, void* stream) {
    int rc = check_shape(shape);
    if (rc) return rc;
    if (!workspace || !out_bf16) return VMOE_ERR_NULL;
    if (M < 0 || M > shape->max_tokens) return VMOE_ERR_SHAPE;
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    return launch_combine(*shape, M, ws, static_cast<__nv_bfloat16*>(out_bf16), static_cast<cudaStream_t>(stream));
}

int vmoe_forward(const vmoe_shape* shape, const vmoe_weights* routed, const vmoe_weights* shared,
                 const void* hidden_bf16, const float* router_logits, const int32_t* topk_ids,
                 const float* topk_weights, const int32_t* expert_map, void* out_bf16, int32_t M,
                 void* workspace, size_t workspace_bytes, void* stream) {
    return vmoe_forward_ex(shape, routed, shared, hidden_bf16, router_logits, topk_ids, topk_weights, expert_map,
                           out_bf16, M, workspace, workspace_bytes, nullptr, stream);
}

int vmoe_router_gemv(const void* hidden_bf16, const void* gate_weight, int32_t gate_dtype,
                     int32_t M, int32_t K, int32_t E, float* logits, void* stream) {
    if (!hidden_bf16 || !gate_weight || !logits) return M == 0 ? VMOE_OK : VMOE_ERR_NULL;
    if (M < 0) return VMOE_ERR_SHAPE;
    if (!aligned16(hidden_bf16) || !aligned16(gate_weight)) return VMOE_ERR_ALIGN;
    return launch_router_gemv(static_cast<const __nv_bfloat16*>(hidden_bf16), gate_weight, gate_dtype, M, K, E, logits,
                              static_cast<cudaStream_t>(stream));
}

int vmoe_forward_ex(const vmoe_shape* shape, const vmoe_weights* routed, const vmoe_weights* shared,
                    const void* hidden_bf16, const float* router_logits, const int32_t* topk_ids,
                    const float* topk_weights, const int32_t* expert_map, void* out_bf16, int32_t M,
                    void* workspace, size_t workspace_bytes, const vmoe_extras* extras, void* stream) {
    int rc = check_call(shape, routed, shared, M, workspace);
    if (rc) return rc;
    if (M == 0) return VMOE_OK;                          // an empty batch may come with NULL data pointers
    const void* gate_weight = extras ? extras->gate_weight : nullptr;
    const __nv_bfloat16* residual = extras ? static_cast<const __nv_bfloat16*>(extras->residual_bf16) : nullptr;
    const uint8_t* pre_q = extras ? extras->hidden_q : nullptr;
    const uint8_t* pre_sf = extras ? extras->hidden_sf : nullptr;
    const float* norm_w = extras ? extras->next_norm_weight : nullptr;
    if ((pre_q == nullptr) != (pre_sf == nullptr)) return VMOE_ERR_NULL;
    if (norm_w && (!extras->next_act_q || !extras->next_act_sf)) return VMOE_ERR_NULL;
    const bool own_logits = !router_logits && !(topk_ids && topk_weights) && gate_weight;
    if (!out_bf16 || (!hidden_bf16 && (!pre_q || own_logits))) return VMOE_ERR_NULL;
    if (!router_logits && !(topk_ids && topk_weights) && !gate_weight) return VMOE_ERR_NULL;
    if ((hidden_bf16 && !aligned16(hidden_bf16)) || !aligned16(out_bf16) || (residual && !aligned16(residual))) return VMOE_ERR_ALIGN;
    if (pre_q && ((reinterpret_cast<uintptr_t>(pre_q) & 7) != 0)) return VMOE_ERR_ALIGN;
    if (norm_w && ((reinterpret_cast<uintptr_t>(extras->next_act_q) & 7) != 0 ||
                   (extras->next_normed_bf16 && !aligned16(extras->next_normed_bf16)))) return VMOE_ERR_ALIGN;
    if (own_logits && !aligned16(gate_weight)) return VMOE_ERR_ALIGN;
    if (own_logits && shape->num_global_experts > (shape->topk + 1) * shape->hidden) return VMOE_ERR_SHAPE;   // logits scratch
    if (workspace_bytes < vmoe_workspace_bytes(shape)) return VMOE_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    Workspace ws;
    if ((rc = resolve_workspace(shape, workspace, &ws))) return rc;
    const WeightSet r = to_set(routed), sh = to_set(shape->has_shared ? shared : nullptr);
    if (own_logits) {
        // the logits live in the (still unused) down-projection output buffer until the router has read them
        float* lg = ws.pair_out;
        if ((rc = launch_router_gemv(static_cast<const __nv_bfloat16*>(hidden_bf16), gate_weight, extras->gate_dtype, M,
                                     shape->hidden, shape->num_global_experts, lg, st))) return rc;
        router_logits = lg;
    }
    int path;
    if ((rc = pick_path(shape, routed, shared, &path))) return rc;
    const int cap = tc_unit_cap(*shape, M);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(out_bf16);
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(hidden_bf16);
    // small batches: router + tables (+ quantiser) in one CTA
    bool front = false;
    if (path == VMOE_PATH_TC && cap == TC_UNIT_TOK_SMALL) {
        if ((rc = launch_front(*shape, router_logits, topk_ids, topk_weights, expert_map, M, ws, st, cap, &front)))
            return rc;
        if (front && router_logits) { topk_ids = ws.topk_ids; topk_weights = ws.topk_weights; }
    }
    if (!front) {
        if (router_logits) {
            if ((rc = launch_route(router_logits, M, shape->num_global_experts, shape->topk, ws.topk_ids,
                                   ws.topk_weights, st))) return rc;
            topk_ids = ws.topk_ids; topk_weights = ws.topk_weights;
        }
        if ((rc = launch_tables(*shape, topk_ids, topk_weights, expert_map, M, ws, st, cap, path != VMOE_PATH_TC))) return rc;
    }
    if (path == VMOE_PATH_TC) {
        const PreparedSet prep = to_prep(routed, shape->has_shared ? shared : nullptr);
        // small batches: the permuting quantiser is the first work of the fused kernel; large ones: its own launch
        const TcQuant quant{x, pre_q, pre_sf, topk_ids, expert_map};
        const bool in_kernel = cap == TC_UNIT_TOK_SMALL && tuning("VMOE_FUSE_QUANT", 1) != 0 && tuning("VMOE_FUSE_PHASES", 1) != 0;
        if (!in_kernel && (rc = launch_permute_quantize(*shape, x, topk_ids, expert_map, M, ws, st, pre_q, pre_sf))) return rc;
        bool combined = false;
        // VMOE_PAIR_ROWS_BF16=1 (large batches, plain combine only): the down projection stores its per-pair rows as
        // bf16 and the combine sums them in fp32 in the same fixed order -- half the bytes of that round trip for a
        // second rounding per pair.  Off by default: the default path keeps fp32 rows.
        if (cap == TC_UNIT_TOK_PREFILL && !norm_w && tuning("VMOE_PAIR_ROWS_BF16", 0) != 0) ws.pair_rows_bf16 = 1;
        // with the next layer's RMSNorm behind it the combine runs as its own row-wide kernel
        if ((rc = launch_tc(*shape, r, sh, prep, M, ws, st, TC_PHASE_GATE_UP | TC_PHASE_DOWN, norm_w ? nullptr : out, residual, &combined,
                            -1, -1, nullptr, in_kernel ? &quant : nullptr))) return rc;
        if (combined) return VMOE_OK;
    } else {
        if (pre_q) {
            if (cudaMemcpyAsync(ws.act_q, pre_q, (size_t)M * shape->hidden / 2, cudaMemcpyDeviceToDevice, st) != cudaSuccess ||
                cudaMemcpyAsync(ws.act_sf, pre_sf, (size_t)M * shape->hidden / 16, cudaMemcpyDeviceToDevice, st) != cudaSuccess) return VMOE_ERR_CUDA;
        } else if ((rc = launch_quantize(x, M, shape->hidden, ws.act_q, ws.act_sf, st))) return rc;
        if ((rc = launch_gate_up(*shape, r, sh, M, ws, st))) return rc;
        if ((rc = launch_down(*shape, r, sh, M, ws, st))) return rc;
    }
    if (norm_w)
        return launch_combine_norm(*shape, M, ws, out, st, residual, norm_w, extras->next_norm_eps,
                                   static_cast<__nv_bfloat16*>(extras->next_normed_bf16), extras->next_act_q, extras->next_act_sf);
    return launch_combine(*shape, M, ws, out, st, residual);
}

int vmoe_rmsnorm_quantize(const void* x_bf16, const float* gamma, float eps, int32_t rows, int32_t K,
                          void* y_bf16, uint8_t* packed, uint8_t* sf, void* stream) {
    if (rows == 0) return VMOE_OK;
    if (!x_bf16 || !gamma || !packed || !sf) return VMOE_ERR_NULL;
    if (rows < 0 || K <= 0 || K % SF_BLOCK) return VMOE_ERR_SHAPE;
    if (!aligned16(x_bf16) || (y_bf16 && !aligned16(y_bf16)) || (reinterpret_cast<uintptr_t>(packed) & 7)) return VMOE_ERR_ALIGN;
    return launch_rmsnorm_quantize(static_cast<const __nv_bfloat16*>(x_bf16), gamma, eps, rows, K,
                                   static_cast<__nv_bfloat16*>(y_bf16), packed, sf, static_cast<cudaStream_t>(stream));
}

int vmoe_read_status(void* workspace, const vmoe_shape* shape, void* stream) {
    Workspace ws;
    int rc = resolve_workspace(shape, workspace, &ws);
    if (rc) return rc;
    int32_t v = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&v, ws.counters + CNT_STATUS, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return VMOE_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return VMOE_ERR_CUDA;
    if (v != 0) cudaMemsetAsync(ws.counters + CNT_STATUS, 0, 4, st);
    return v;
}

}  // extern "C"
