// Router (softmax + top-k + renormalise) and the permutation of pairs by expert.
//
// Router semantics: fused-moe/csrc/megakernel_v1.cu:491-537 of the reference (fp32 softmax,
// strict '>' selection so the lowest expert id wins a tie, descending order, renormalise).
// Permutation semantics: fused-moe/csrc/verdict_fused_grouped.cu:655-691 (stable sort of the
// token-major pairs by expert id, expert offsets, gather indices, scatter weights).
#include "vmoe_common.cuh"

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
    float* p = s_prob + (size_t)warp * E;
    const float* l = logits + (size_t)m * E;

    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) { float v = l[e]; p[e] = v; mx = fmaxf(mx, v); }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { float v = expf(p[e] - mx); p[e] = v; sum += v; }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) p[e] *= inv;
    __syncwarp();

    float sel_w = 0.f; int sel_id = 0; float wsum = 0.f;   // lane j keeps the j-th selection
    for (int j = 0; j < T; ++j) {
        float bv = -1.0f; int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { float v = p[e]; if (v > bv) { bv = v; bi = e; } }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int   oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == j) { sel_w = bv; sel_id = bi; }
        if (lane == 0) p[bi] = -2.0f;            // taken
        wsum += bv;                              // same value in every lane, rank order
        __syncwarp();
    }
    const float winv = 1.0f / wsum;
    if (lane < T) {
        topk_ids[(size_t)m * T + lane] = sel_id;
        topk_w[(size_t)m * T + lane] = sel_w * winv;
    }
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
struct TableArgs {
    const int32_t* ids; const float* w; const int32_t* expert_map;
    int M, T, E, has_shared, words;   // words = ceil(M / 32)
    int tc_cap;                       // tokens per tensor-core unit
    int gemv_units;                   // also emit the 4-token work units of the CUDA-core path
    Workspace ws;
};

__device__ __forceinline__ int local_expert(const TableArgs& a, int p) {
    int e = a.ids[p];
    if (a.expert_map) e = a.expert_map[e];
    return (e >= 0 && e < a.E) ? e : -1;
}

__device__ void phase_clear(const TableArgs& a, int tid, int nthr) {
    const int n = a.E * a.words;
    for (int i = tid; i < n; i += nthr) a.ws.bitmap[i] = 0u;
    if (tid < CNT_N && tid != CNT_STATUS) a.ws.counters[tid] = 0;
}
__device__ void phase_mark(const TableArgs& a, int tid, int nthr) {
    const int P = a.M * a.T;
    for (int p = tid; p < P; p += nthr) {
        const int e = local_expert(a, p);
        if (e >= 0) { const int m = p / a.T; atomicOr(&a.ws.bitmap[(size_t)e * a.words + (m >> 5)], 1u << (m & 31)); }
    }
}
// Running popcount per bitmap word and the pair count per expert.  A warp takes 32 / wp experts at a
// time (wp = words rounded up to a power of two) with a segmented shuffle scan over each expert's
// words; experts with more than 32 words are walked 32 words at a time by a whole warp.
__device__ void phase_count(const TableArgs& a, int warp, int nwarps, int lane, int32_t* s_count) {
    if (a.words <= 32) {
        int wp = 1;
        while (wp < a.words) wp <<= 1;
        const int gpw = 32 / wp, sub = lane / wp, wl = lane % wp;
        for (int e0 = warp * gpw; e0 < a.E; e0 += nwarps * gpw) {
            const int e = e0 + sub;
            const bool valid = e < a.E && wl < a.words;
            const int c = valid ? __popc(a.ws.bitmap[(size_t)e * a.words + wl]) : 0;
            int incl = c;
            for (int o = 1; o < wp; o <<= 1) { const int t = __shfl_up_sync(0xffffffffu, incl, o, wp); if (wl >= o) incl += t; }
            if (valid) a.ws.word_prefix[(size_t)e * a.words + wl] = incl - c;
            if (wl == wp - 1 && e < a.E) s_count[e] = incl;
        }
        return;
    }
    for (int e = warp; e < a.E; e += nwarps) {
        int running = 0;
        for (int w0 = 0; w0 < a.words; w0 += 32) {
            const int w = w0 + lane;
            const int c = (w < a.words) ? __popc(a.ws.bitmap[(size_t)e * a.words + w]) : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { int t = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += t; }
            if (w < a.words) a.ws.word_prefix[(size_t)e * a.words + w] = running + incl - c;
            running += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) s_count[e] = running;
    }
}
// single CTA: exclusive scan of counts -> expert_offsets, GEMV unit list, tensor-core unit list
__device__ __forceinline__ int tc_box(int n) { return n <= 8 ? 8 : n <= 16 ? 16 : n <= 32 ? 32 : 64; }
__device__ void phase_scan(const TableArgs& a, int tid, int nthr, const int32_t* s_count, int32_t* s_scan) {
    // chunked serial-per-thread scan: thread i owns experts [i*per, (i+1)*per)
    const int n = a.E + (a.has_shared ? 1 : 0);
    const int per = (n + nthr - 1) / nthr;
    int csum = 0, usum = 0, tsum = 0;
    for (int k = 0; k < per; ++k) {
        const int e = tid * per + k;
        if (e < n) {
            const int c = (e < a.E) ? s_count[e] : a.M;
            csum += c; usum += (c + TOK_PER_UNIT - 1) / TOK_PER_UNIT; tsum += (c + a.tc_cap - 1) / a.tc_cap;
        }
    }
    // two-level exclusive scan of the per-thread sums: inside each warp, then over the warp totals
    const int lane = tid & 31, wid = tid >> 5, nw = (nthr + 31) >> 5;
    int ci = csum, ui = usum, ti = tsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int c2 = __shfl_up_sync(0xffffffffu, ci, o), u2 = __shfl_up_sync(0xffffffffu, ui, o), t2 = __shfl_up_sync(0xffffffffu, ti, o);
        if (lane >= o) { ci += c2; ui += u2; ti += t2; }
    }
    if (lane == 31) { s_scan[wid] = ci; s_scan[32 + wid] = ui; s_scan[64 + wid] = ti; }
    __syncthreads();
    if (tid < 32) {
        const int c0 = tid < nw ? s_scan[tid] : 0, u0 = tid < nw ? s_scan[32 + tid] : 0, t0 = tid < nw ? s_scan[64 + tid] : 0;
        int cw = c0, uw = u0, tw = t0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int c2 = __shfl_up_sync(0xffffffffu, cw, o), u2 = __shfl_up_sync(0xffffffffu, uw, o), t2 = __shfl_up_sync(0xffffffffu, tw, o);
            if (tid >= o) { cw += c2; uw += u2; tw += t2; }
        }
        s_scan[tid] = cw - c0; s_scan[32 + tid] = uw - u0; s_scan[64 + tid] = tw - t0;     // exclusive warp bases
        if (tid == 31) {
            a.ws.counters[CNT_UNITS] = a.gemv_units ? uw : 0; a.ws.counters[CNT_SLOTS] = cw; a.ws.counters[CNT_TC_UNITS] = tw;
            a.ws.expert_offsets[n] = cw;
            if (!a.has_shared) a.ws.expert_offsets[n + 1] = cw;
        }
    }
    __syncthreads();
    int c = s_scan[wid] + ci - csum, u = s_scan[32 + wid] + ui - usum, t = s_scan[64 + wid] + ti - tsum;
    for (int k = 0; k < per; ++k) {
        const int e = tid * per + k;
        if (e < n) {
            const int cnt = (e < a.E) ? s_count[e] : a.M;
            a.ws.expert_offsets[e] = c;
            if (a.gemv_units)
                for (int s = 0; s < cnt; s += TOK_PER_UNIT)
                    a.ws.units[u++] = make_int4(e, c + s, min(TOK_PER_UNIT, cnt - s), 0);
            if (a.ws.tc_units) {
                a.ws.tc_unit_base[e] = t;
                for (int s = 0; s < cnt; s += a.tc_cap) {
                    const int nt = min(a.tc_cap, cnt - s);
                    a.ws.tc_units[t++] = make_int4(e, c + s, nt, tc_box(nt));
                }
            }
            c += cnt;
        }
    }
}
__device__ void phase_place(const TableArgs& a, int tid, int nthr) {
    const int P = a.M * a.T;
    for (int p = tid; p < P; p += nthr) {
        const int e = local_expert(a, p);
        int slot = -1;
        if (e >= 0) {
            const int m = p / a.T;
            const size_t wi = (size_t)e * a.words + (m >> 5);
            slot = a.ws.expert_offsets[e] + a.ws.word_prefix[wi] + __popc(a.ws.bitmap[wi] & ((1u << (m & 31)) - 1u));
            a.ws.sorted_pair[slot] = p;
            a.ws.gather_idx[slot] = m;
            a.ws.scatter_weights[slot] = a.w[p];
        }
        a.ws.pair_slot[p] = slot;
    }
    if (a.has_shared) {
        const int base = a.ws.expert_offsets[a.E];
        for (int m = tid; m < a.M; m += nthr) {
            a.ws.sorted_pair[base + m] = P + m;
            a.ws.gather_idx[base + m] = m;
            a.ws.scatter_weights[base + m] = 1.0f;
        }
    }
}

constexpr int TABLE_THREADS = 1024;

// small problems: everything in one CTA
__global__ void __launch_bounds__(TABLE_THREADS) tables_fused_kernel(TableArgs a, int tables_in_smem) {
    extern __shared__ int32_t s_mem[];          // [E] counts + [3 * nthr] scan (+ bitmap and running popcounts)
    int32_t* s_count = s_mem; int32_t* s_scan = s_mem + a.E;
    const int tid = threadIdx.x, nthr = blockDim.x;
    pdl_begin();
    if (tables_in_smem) {
        // the bitmap and its popcounts are touched by every phase: keep them on chip when they fit
        a.ws.bitmap = reinterpret_cast<uint32_t*>(s_scan + 3 * nthr);
        a.ws.word_prefix = reinterpret_cast<int32_t*>(a.ws.bitmap + (size_t)a.E * a.words);
    }
    phase_clear(a, tid, nthr);       __syncthreads();
    phase_mark(a, tid, nthr);        __syncthreads();
    phase_count(a, tid >> 5, nthr >> 5, tid & 31, s_count); __syncthreads();
    phase_scan(a, tid, nthr, s_count, s_scan); __syncthreads();
    phase_place(a, tid, nthr);
}
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

int launch_tables(const vmoe_shape& s, const int32_t* ids, const float* w, const int32_t* expert_map,
                  int M, const Workspace& ws, cudaStream_t st, int tc_cap, bool gemv_units) {
    TableArgs a;
    a.tc_cap = tc_cap;
    a.gemv_units = gemv_units ? 1 : 0;
    a.ids = ids; a.w = w; a.expert_map = expert_map;
    a.M = M; a.T = s.topk; a.E = s.num_experts; a.has_shared = s.has_shared; a.words = (M + 31) / 32;
    a.ws = ws;
    const size_t smem = ((size_t)a.E + 3 * TABLE_THREADS) * sizeof(int32_t);
    if (smem > 200 * 1024) return VMOE_ERR_SHAPE;
    const size_t smem_tab = smem + 2 * (size_t)a.E * a.words * sizeof(int32_t);
    const bool in_smem = smem_tab <= 200 * 1024;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(tables_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done = true;
    }
    if ((long long)M * s.topk <= 16384) {
        launch_pdl(tables_fused_kernel, 1u, (unsigned)TABLE_THREADS, in_smem ? smem_tab : smem, st, a, in_smem ? 1 : 0);
    } else {
        const int blocks = 296;
        launch_pdl(tables_clear_kernel, (unsigned)blocks, 256u, 0, st, a);
        launch_pdl(tables_mark_kernel, (unsigned)blocks, 256u, 0, st, a);
        launch_pdl(tables_count_kernel, (unsigned)((a.E + 7) / 8), 256u, 0, st, a);
        launch_pdl(tables_scan_kernel, 1u, (unsigned)TABLE_THREADS, 0, st, a);
        launch_pdl(tables_place_kernel, (unsigned)blocks, 256u, 0, st, a);
    }
    return cuda_status(cudaGetLastError());
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

// Same phases as tables_fused_kernel, over caller outputs + the static scratch.  The first
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
    a.tc_cap = TC_UNIT_TOK;
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
