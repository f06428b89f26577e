// Router (softmax + top-k + renormalise) and the permutation of pairs by expert.
//
// Router semantics: fused-moe/csrc/megakernel_v1.cu:491-537 of the reference (fp32 softmax,
// strict '>' selection so the lowest expert id wins a tie, descending order, renormalise).
// Permutation semantics: fused-moe/csrc/verdict_fused_grouped.cu:655-691 (stable sort of the
// token-major pairs by expert id, expert offsets, gather indices, scatter weights).
#include "vmoe_common.cuh"
#include "vmoe_phases.cuh"

#include <stdlib.h>

namespace vmoe {

// ---------------------------------------------------------------------------------
// Router: one warp per token.  Probabilities live in shared memory; each of the T
// rounds takes the arg-max under the order (probability desc, expert id asc).
// ---------------------------------------------------------------------------------
constexpr int ROUTE_WARPS = 4;

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_kernel(const float* __restrict__ logits, int M, int E, int T,
             int32_t* __restrict__ topk_ids, float* __restrict__ topk_w) {
    extern __shared__ float s_prob[];            // [ROUTE_WARPS][E]
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m = blockIdx.x * ROUTE_WARPS + warp;
    if (m >= M) return;
    route_token(logits + (size_t)m * E, s_prob + (size_t)warp * E, E, T, lane, topk_ids + (size_t)m * T, topk_w + (size_t)m * T);
}

int launch_route(const float* logits, int M, int E, int T, int32_t* ids, float* w, cudaStream_t st) {
    if (M == 0) return VMOE_OK;
    const size_t smem = (size_t)ROUTE_WARPS * E * sizeof(float);
    if (smem > 200 * 1024) return VMOE_ERR_SHAPE;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(route_kernel, (unsigned)((M + ROUTE_WARPS - 1) / ROUTE_WARPS), ROUTE_WARPS * 32, smem, st, logits, M, E, T, ids, w);
    return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------------
// Permutation by expert.
//
// A token selects an expert at most once, so the stable rank of pair (m, j) inside
// expert e is the number of tokens m' < m that selected e.  Phase A sets bit m of row e
// of an [E, ceil(M/32)] bitmap; phase B gives every expert its pair count, the
// exclusive scan over experts, a running popcount per bitmap word and its share of the
// GEMV work-unit list; phase C places each pair at offset[e] + word_prefix + popc(bits
// below m).  Deterministic, no sorting network, no atomics on the result.
// The always-on shared expert is expert id E: slot range [offset[E], offset[E] + M),
// pair index P + m, weight 1.0.
// ---------------------------------------------------------------------------------
constexpr int TABLE_THREADS = 1024;

// large problems: grid-wide phases as separate launches
__global__ void tables_clear_kernel(TableArgs a) { pdl_begin(); phase_clear(a, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x); }
__global__ void tables_mark_kernel(TableArgs a)  { pdl_begin(); phase_mark(a, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x); }
// counts go through expert_offsets (each entry is read by its owner before the scan overwrites it)
__global__ void __launch_bounds__(256) tables_count_kernel(TableArgs a) {
    pdl_begin();
    phase_count(a, (blockIdx.x * blockDim.x + threadIdx.x) >> 5, (gridDim.x * blockDim.x) >> 5, threadIdx.x & 31, a.ws.expert_offsets);
}
__global__ void __launch_bounds__(TABLE_THREADS) tables_scan_kernel(TableArgs a) {
    __shared__ int32_t s_scan[96];
    pdl_begin();
    phase_scan(a, threadIdx.x, blockDim.x, a.ws.expert_offsets, s_scan);
}
__global__ void tables_place_kernel(TableArgs a) { pdl_begin(); phase_place(a, blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x); }

// ---------------------------------------------------------------------------------
// Up to 4096 pairs: the front of the layer in ONE CTA.  Optionally the router (one warp per token), then the
// permutation phases.  Everything a later phase of this CTA reads back (ids, weights, expert
// offsets, first unit per expert, slot of each pair; bitmap and running popcounts when they fit) lives in
// shared memory and is copied to the workspace at the end, so no phase waits for a round trip through L2.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(TABLE_THREADS)
front_kernel(const float* __restrict__ logits, int num_global, TableArgs a, int tables_in_smem) {
    extern __shared__ int32_t s_mem[];
    const int tid = threadIdx.x, nthr = blockDim.x, warp = tid >> 5, lane = tid & 31, nwarps = nthr >> 5;
    const int P = a.M * a.T;
    int32_t* s_count = s_mem;                      // [E]
    int32_t* s_scan = s_count + a.E;               // [3 * nthr]
    int32_t* s_off = s_scan + 3 * nthr;            // [E + 2] expert offsets
    int32_t* s_ub = s_off + a.E + 2;               // [E + 2] first tensor-core unit per expert
    int32_t* s_slot = s_ub + a.E + 2;              // [P] slot of each pair
    int32_t* s_ids = s_slot + P;                   // [P]
    float* s_w = reinterpret_cast<float*>(s_ids + P);      // [P]
    int32_t* s_next = s_ids + 2 * P;
    pdl_begin();
    if (tables_in_smem) {
        a.ws.bitmap = reinterpret_cast<uint32_t*>(s_next);
        a.ws.word_prefix = s_next + (size_t)a.E * a.words;
        s_next += 2 * (size_t)a.E * a.words;
    }
    if (logits) {
        float* s_prob = reinterpret_cast<float*>(s_next) + (size_t)warp * num_global;
        for (int m = warp; m < a.M; m += nwarps) {
            route_token(logits + (size_t)m * num_global, s_prob, num_global, a.T, lane, s_ids + m * a.T, s_w + m * a.T);
            __syncwarp();
            if (lane < a.T) {        // the workspace copy (read by later kernels and by the caller)
                a.ws.topk_ids[(size_t)m * a.T + lane] = s_ids[m * a.T + lane];
                a.ws.topk_weights[(size_t)m * a.T + lane] = s_w[m * a.T + lane];
            }
        }
    } else {
        for (int p = tid; p < P; p += nthr) { s_ids[p] = a.ids[p]; s_w[p] = a.w[p]; }
    }
    for (int i = tid; i < a.E + 2; i += nthr) s_ub[i] = 0;
    int32_t* g_off = a.ws.expert_offsets; int32_t* g_ub = a.ws.tc_unit_base; int32_t* g_slot = a.ws.pair_slot;
    a.ids = s_ids; a.w = s_w;
    a.ws.expert_offsets = s_off; a.ws.tc_unit_base = s_ub; a.ws.pair_slot = s_slot;
    phase_clear(a, tid, nthr);       // touches nothing the router reads or writes: runs beside it on the other warps
    __syncthreads();
    phase_mark(a, tid, nthr);        __syncthreads();
    phase_count(a, warp, nwarps, lane, s_count); __syncthreads();
    phase_scan(a, tid, nthr, s_count, s_scan); __syncthreads();
    phase_place(a, tid, nthr);
    __syncthreads();
    for (int i = tid; i < a.E + 2; i += nthr) g_off[i] = s_off[i];
    if (g_ub) for (int i = tid; i < a.E + 1; i += nthr) g_ub[i] = s_ub[i];
    for (int p = tid; p < P; p += nthr) g_slot[p] = s_slot[p];
}

int tuning(const char* name, int dflt) {
    const char* v = getenv(name);
    return v ? atoi(v) : dflt;
}

// Launches front_kernel when the problem fits one CTA; *done = false (and nothing launched) otherwise.
static int launch_one_cta(const vmoe_shape& s, const float* logits, const int32_t* ids, const float* w,
                          const int32_t* expert_map, int M, const Workspace& ws,
                          cudaStream_t st, int tc_cap, bool gemv_units, bool* done) {
    *done = false;
    const long long P = (long long)M * s.topk;
    if (M <= 0 || P > 4096) return VMOE_OK;
    const int nthr = TABLE_THREADS;
    TableArgs a;
    a.tc_cap = tc_cap; a.gemv_units = gemv_units ? 1 : 0;
    a.ids = ids; a.w = w; a.expert_map = expert_map;
    a.M = M; a.T = s.topk; a.E = s.num_experts; a.has_shared = s.has_shared; a.words = (M + 31) / 32;
    a.num_global = s.num_global_experts;
    a.tiles_d = s.hidden / TC_TILE_ROWS;
    a.ws = ws;
    size_t smem = ((size_t)a.E + 3 * nthr + 2 * ((size_t)a.E + 2) + 3 * (size_t)P) * sizeof(int32_t);
    const size_t tab = 2 * (size_t)a.E * a.words * sizeof(int32_t);
    const size_t prob = logits ? (size_t)(nthr / 32) * s.num_global_experts * sizeof(float) : 0;
    const bool in_smem = smem + tab + prob <= 200 * 1024;
    if (in_smem) smem += tab;
    smem += prob;
    if (smem > 200 * 1024) return VMOE_OK;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(front_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done = true;
    }
    launch_pdl(front_kernel, 1u, (unsigned)nthr, smem, st, logits, s.num_global_experts, a, in_smem ? 1 : 0);
    *done = true;
    return cuda_status(cudaGetLastError());
}

int launch_tables(const vmoe_shape& s, const int32_t* ids, const float* w, const int32_t* expert_map,
                  int M, const Workspace& ws, cudaStream_t st, int tc_cap, bool gemv_units) {
    bool done = false;
    int rc = launch_one_cta(s, nullptr, ids, w, expert_map, M, ws, st, tc_cap, gemv_units, &done);
    if (rc || done) return rc;
    // large problems: grid-wide phases as separate launches
    TableArgs a;
    a.tc_cap = tc_cap;
    a.gemv_units = gemv_units ? 1 : 0;
    a.ids = ids; a.w = w; a.expert_map = expert_map;
    a.M = M; a.T = s.topk; a.E = s.num_experts; a.has_shared = s.has_shared; a.words = (M + 31) / 32;
    a.num_global = s.num_global_experts;
    a.tiles_d = s.hidden / TC_TILE_ROWS;
    a.ws = ws;
    const int blocks = 296;
    launch_pdl(tables_clear_kernel, (unsigned)blocks, 256u, 0, st, a);
    launch_pdl(tables_mark_kernel, (unsigned)blocks, 256u, 0, st, a);
    launch_pdl(tables_count_kernel, (unsigned)((a.E + 7) / 8), 256u, 0, st, a);
    launch_pdl(tables_scan_kernel, 1u, (unsigned)TABLE_THREADS, 0, st, a);
    launch_pdl(tables_place_kernel, (unsigned)blocks, 256u, 0, st, a);
    return cuda_status(cudaGetLastError());
}

int launch_front(const vmoe_shape& s, const float* logits, const int32_t* ids, const float* w,
                 const int32_t* expert_map, int M, const Workspace& ws, cudaStream_t st, int tc_cap, bool* done) {
    const int max_tokens = tuning("VMOE_FRONT_TOKENS", 32);            // router inside the one-CTA front up to this batch
    *done = false;
    if (M <= 0 || M > max_tokens) return VMOE_OK;
    return launch_one_cta(s, logits, ids, w, expert_map, M, ws, st, tc_cap, false, done);
}

}  // namespace vmoe

namespace vmoe {

// ---------------------------------------------------------------------------------
// vmoe_permute_noalloc: the permutation for callers that cannot obtain device memory.
//
// Some hosts of this library are handed a fixed set of input and output buffers and have
// no way to get one more byte of device memory at the point of the call: a serving worker
// whose memory pool was sized to fill the GPU (a cudaMalloc there fails or steals from the
// KV cache), or a thin C / FFI binding that owns no allocator at all.  For them the scratch
// of the permutation (the expert x token bitmap, its running popcounts, the work-unit list
// and the counters) lives in the file-scope array below instead of a caller-owned workspace.
// The array exists once per GPU that loads the library and stays until the process exits;
// its size fixes the largest problem the entry point accepts.
// ---------------------------------------------------------------------------------
constexpr int NOALLOC_MAX_TOKENS  = 1024;   // M
constexpr int NOALLOC_MAX_EXPERTS = 1024;   // local experts E
constexpr int NOALLOC_WORDS       = NOALLOC_MAX_TOKENS / 32;
constexpr size_t NOALLOC_BITMAP_BYTES = (size_t)NOALLOC_MAX_EXPERTS * NOALLOC_WORDS * 4;          // 128 KiB
constexpr size_t NOALLOC_UNITS = NOALLOC_MAX_EXPERTS + 1 + ((size_t)NOALLOC_MAX_TOKENS * (MAX_TOPK + 1) + TOK_PER_UNIT - 1) / TOK_PER_UNIT;
constexpr size_t NOALLOC_OFF_PREFIX   = NOALLOC_BITMAP_BYTES;
constexpr size_t NOALLOC_OFF_UNITS    = 2 * NOALLOC_BITMAP_BYTES;
constexpr size_t NOALLOC_OFF_COUNTERS = NOALLOC_OFF_UNITS + ((NOALLOC_UNITS * 16 + 255) / 256) * 256;
constexpr size_t NOALLOC_SCRATCH_BYTES = NOALLOC_OFF_COUNTERS + 256;                                // ~ 342 KiB

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

// In host code the name g_noalloc_scratch is only a handle for the symbol; the device address
// is looked up once per device (with that device current) and kept here.
constexpr int NOALLOC_MAX_DEVICES = 64;
static unsigned char* g_noalloc_addr[NOALLOC_MAX_DEVICES] = {nullptr};

static int noalloc_scratch_address(unsigned char** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return VMOE_ERR_CUDA;
    if (g_noalloc_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) return VMOE_ERR_CUDA;
        g_noalloc_addr[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_noalloc_addr[dev];
    return VMOE_OK;
}

// Same phases as the one-CTA front, over caller outputs + the static scratch.  The first
// phase clears the bitmap and the counters, so nothing of an earlier call survives.
__global__ void __launch_bounds__(TABLE_THREADS) tables_noalloc_kernel(TableArgs a) {
    extern __shared__ int32_t s_mem[];
    int32_t* s_count = s_mem; int32_t* s_scan = s_mem + a.E;
    const int tid = threadIdx.x, nthr = blockDim.x;
    phase_clear(a, tid, nthr);       __syncthreads();
    phase_mark(a, tid, nthr);        __syncthreads();
    phase_count(a, tid >> 5, nthr >> 5, tid & 31, s_count); __syncthreads();
    phase_scan(a, tid, nthr, s_count, s_scan); __syncthreads();
    phase_place(a, tid, nthr);
}

}  // namespace vmoe

extern "C" int vmoe_permute_noalloc(const int32_t* topk_ids, const float* topk_weights,
                                    const int32_t* expert_map, int32_t M, int32_t T, int32_t E,
                                    int32_t has_shared, int32_t* expert_offsets, int32_t* sorted_pair,
                                    int32_t* pair_slot, int32_t* gather_idx, float* scatter_weights,
                                    void* stream) {
    using namespace vmoe;
    if (!topk_ids || !topk_weights || !expert_offsets || !sorted_pair || !pair_slot || !gather_idx || !scatter_weights)
        return VMOE_ERR_NULL;
    if (M < 0 || T <= 0 || T > MAX_TOPK || E <= 0) return VMOE_ERR_SHAPE;
    if (M > NOALLOC_MAX_TOKENS || E > NOALLOC_MAX_EXPERTS) return VMOE_ERR_LIMIT;
    unsigned char* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc) return rc;
    TableArgs a;
    a.ids = topk_ids; a.w = topk_weights; a.expert_map = expert_map;
    a.M = M; a.T = T; a.E = E; a.has_shared = has_shared ? 1 : 0; a.words = (M + 31) / 32;
    a.num_global = expert_map ? 0x7fffffff : E;      // the length of expert_map is not known here: see vmoe.h
    a.tiles_d = 0;
    a.tc_cap = TC_UNIT_TOK_SMALL;
    a.gemv_units = 1;
    a.ws = Workspace{};
    a.ws.expert_offsets = expert_offsets; a.ws.sorted_pair = sorted_pair; a.ws.pair_slot = pair_slot;
    a.ws.gather_idx = gather_idx; a.ws.scatter_weights = scatter_weights;
    a.ws.bitmap      = reinterpret_cast<uint32_t*>(scratch);
    a.ws.word_prefix = reinterpret_cast<int32_t*>(scratch + NOALLOC_OFF_PREFIX);
    a.ws.units       = reinterpret_cast<int4*>(scratch + NOALLOC_OFF_UNITS);
    a.ws.counters    = reinterpret_cast<int32_t*>(scratch + NOALLOC_OFF_COUNTERS);
    const size_t smem = ((size_t)E + 3 * TABLE_THREADS) * sizeof(int32_t);   // 16 KiB at the maximum E
    tables_noalloc_kernel<<<1, TABLE_THREADS, smem, static_cast<cudaStream_t>(stream)>>>(a);
    return cuda_status(cudaGetLastError());
}
