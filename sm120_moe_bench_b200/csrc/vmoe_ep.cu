// Expert parallelism inside one NVLink / NVSwitch box: token dispatch and weighted combine as
// peer-memory kernels.  One process per GPU; NCCL (or any other channel) is only used by the host
// to exchange the IPC handles of the slabs once.
//
// Reference semantics: experts in contiguous blocks, gpu = e / (E / G), local = e % (E / G)
// (fused-moe/p2p_moe_routing.py:26-33); the reference itself only sketches the exchange
// (fused-moe/p2p_moe_routing.py:113-131) or replicates every token on every rank and all-reduces
// (fused-moe/patches/p2p_ep_communicator.py:99-155).  Here each token row crosses NVLink once per
// pair, already quantised (2304 bytes at K = 4096), and each weighted output row crosses once
// (fp32, so the owner's fixed-order sum is bit-identical to the single-GPU result).
//
// Per forward call on rank r (one stream, no host synchronisation, five launches; eight around the token-major kernels):
//   1 router    one warp per local token
//   2 dispatch  one CTA per token: the plan (destination rank and position inside the (source -> destination)
//               slab of every pair, in pair order: deterministic), then each 16-block quantised once and stored
//               into the slab of every destination of the token (16-byte peer stores); the last CTA publishes
//               row counts and the call flag on every peer
//   3 gather    one CTA: bounded acquire-wait on every source's flag, dense list of the rows that actually
//               arrived (prefix over the sources' counts), permutation tables over exactly those rows
//   4 permute   received rows into sorted-slot order + scale atoms, destination pointer of every output row: the
//               first work of the weights-as-rows kernel (a launch of its own in front of the token-major kernels)
//   5 experts   the tcgen05 kernels of the single-GPU layer; the down projection's epilogue stores each
//               weighted row straight into the token owner's combine slab over NVLink (128 contiguous bytes of
//               a row per store instruction); the last CTA
//               publishes the "rows are in place" flag on every peer (a one-warp launch behind the token-major kernels)
//   6 combine   bounded wait on every rank's flag, fixed-order sum (+ residual) -> bf16; the last CTA
//               advances the call counter
// The call number lives in device memory (a counter in the workspace, advanced by step 6), so the chain has
// no per-call host argument and can be captured in a CUDA graph and replayed.  Every flag carries the call
// number and an error bit: a rank that ran into a time-out or a capacity overflow still signals, marked,
// and every rank that sees a marked flag reports VMOE_ERR_PEER and leaves its output unwritten.
// Plain peer loads / stores only: no multimem, no TMA from peer memory.
#include "vmoe_common.cuh"
#include "vmoe_phases.cuh"

#include <string.h>

namespace vmoe {

constexpr int EP_MAX_RANKS = 16;

struct EpFlags {            // lives at the start of every rank's slab; written by peers
    int32_t dispatch_flag[EP_MAX_RANKS];    // [src] 2 * call + error bit of the last completed dispatch from src
    int32_t dispatch_count[EP_MAX_RANKS];   // [src] rows src wrote for that call
    int32_t combine_flag[EP_MAX_RANKS];     // [src] 2 * call + error bit of the last completed down projection on src
    int32_t pad[16];
};

struct EpLayout {           // byte offsets inside a slab; identical on every rank
    size_t flags, recv_q, recv_sf, recv_meta, comb, total;
};

static size_t ep_align(size_t v) { return (v + 255) / 256 * 256; }

static EpLayout ep_layout(int world, int capacity, int max_local_tokens, int K, int T) {
    EpLayout L;
    size_t off = 0;
    auto take = [&](size_t b) { size_t o = off; off = ep_align(off + b); return o; };
    L.flags = take(sizeof(EpFlags));
    L.recv_q = take((size_t)world * capacity * (K / 2));
    L.recv_sf = take((size_t)world * capacity * (K / 16));
    L.recv_meta = take((size_t)world * capacity * 16);
    L.comb = take((size_t)max_local_tokens * (T + 1) * K * 4);
    L.total = off;
    return L;
}

// device-side state of the exchange (local workspace, behind the regular workspace)
struct EpState {
    int32_t epoch;              // calls completed on this rank
    int32_t ticket_dispatch, ticket_experts, ticket_combine;
    int32_t recv_rows;          // rows that arrived for this call
    int32_t src_base[EP_MAX_RANKS + 1];   // exclusive prefix of the rows per source
};

struct EpDev {              // by value into kernels
    int rank, world, e_local, capacity;
    unsigned long long wait_ns;             // limit of every cross-GPU wait
    uint8_t* slab[EP_MAX_RANKS];            // every rank's slab as mapped into this process
    EpLayout L;
    EpState* state;
    int32_t* flat_ids; float* flat_w; float** row_dst;
    unsigned long long* timeline;           // development builds (-DVMOE_TIMELINE) only
};
#ifdef VMOE_TIMELINE
#define EP_MARK_MIN(ep, slot) do { if ((ep).timeline) atomicMin(&(ep).timeline[slot], global_timer_ns()); } while (0)
#define EP_MARK_MAX(ep, slot) do { if ((ep).timeline) atomicMax(&(ep).timeline[slot], global_timer_ns()); } while (0)
#else
#define EP_MARK_MIN(ep, slot) ((void)0)
#define EP_MARK_MAX(ep, slot) ((void)0)
#endif

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until the flag carries call number `call` (or a later one).  Returns the flag value, or -1
// when the limit passes.
__device__ __forceinline__ int32_t wait_flag(const int32_t* p, int32_t call, unsigned long long limit_ns) {
    int32_t v = ld_acquire_sys(p);
    if ((v >> 1) >= call) return v;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        v = ld_acquire_sys(p);
        if ((v >> 1) >= call) return v;
        if ((i & 15u) == 0 && global_timer_ns() - t0 > limit_ns) return -1;
    }
}

// ---------------------------------------------------------------------------------
// 2 dispatch: one CTA per local token.  The CTA first works out where the token's rows go -- destination rank of
// every pair and its position inside the (this rank -> destination) slab, which is the number of earlier pairs, in pair
// order, with the same destination: pair p = m*T + j for routed pairs, M*T + m for the shared expert, which stays
// on the owner (deterministic: a count over the ids in front, no atomics on the result) -- then quantises each
// 16-block of the row once (same arithmetic as quantize_kernel) and stores it into the slab of every destination
// (16-byte peer stores).  The last CTA to finish releases the row counts and the call flag on every peer.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   const float* __restrict__ topk_w, int M, int K, int T, int has_shared, EpDev ep,
                   int32_t* status) {
    __shared__ int32_t s_before[EP_MAX_RANKS];      // routed pairs of earlier tokens per destination
    __shared__ int32_t s_total[EP_MAX_RANKS];       // routed pairs of all tokens per destination
    __shared__ int32_t s_dst[MAX_TOPK + 1], s_pos[MAX_TOPK + 1];
    __shared__ __align__(16) uint8_t s_sf[256];        // block scales of one chunk of 256 blocks
    __shared__ int s_last;
    if (threadIdx.x == 0) EP_MARK_MIN(ep, 20);
    pdl_begin();
    if (threadIdx.x == 0) EP_MARK_MIN(ep, 21);
    const int tid = threadIdx.x, m = blockIdx.x;
    if (tid < EP_MAX_RANKS) { s_before[tid] = 0; s_total[tid] = 0; }
    __syncthreads();
    const int P = M * T;
    for (int p0 = 0; p0 < P; p0 += blockDim.x) {            // counted by ballots: one shared-memory atomic per warp and destination
        const int p = p0 + tid;
        const int d = p < P ? min(max(topk_ids[p] / ep.e_local, 0), ep.world - 1) : -1;
        for (int dd = 0; dd < ep.world; ++dd) {
            const unsigned all = __ballot_sync(0xffffffffu, d == dd);
            const unsigned before = __ballot_sync(0xffffffffu, d == dd && p < m * T);
            if ((tid & 31) == 0 && all) {
                atomicAdd(&s_total[dd], __popc(all));
                if (before) atomicAdd(&s_before[dd], __popc(before));
            }
        }
    }
    __syncthreads();
    if (m < M && tid <= T) {
        int d, pos;
        if (tid < T) {
            d = min(max(topk_ids[m * T + tid] / ep.e_local, 0), ep.world - 1);
            pos = s_before[d];
            for (int j = 0; j < tid; ++j) pos += (min(max(topk_ids[m * T + j] / ep.e_local, 0), ep.world - 1) == d);
        } else {
            d = has_shared ? ep.rank : -1;
            pos = s_total[ep.rank] + m;                 // behind every routed pair that stays on this rank
        }
        s_dst[tid] = d; s_pos[tid] = pos;
        if (d >= 0 && pos >= ep.capacity) atomicExch(status, VMOE_ERR_LIMIT);
    }
    __syncthreads();
    if (m < M) {
        const int bpr = K / SF_BLOCK;
        for (int kb0 = 0; kb0 < bpr; kb0 += blockDim.x) {           // uniform trip count: the CTA meets at barriers inside
            const int kb = kb0 + tid;
            if (kb < bpr) {
                const uint4* src = reinterpret_cast<const uint4*>(x + ((size_t)m * bpr + kb) * SF_BLOCK);
                uint4 raw[2] = {src[0], src[1]};
                float v[SF_BLOCK]; uint32_t lo, hi; uint8_t sb;
                quantize_block16(reinterpret_cast<const __nv_bfloat16*>(raw), v, lo, hi, sb);
                s_sf[tid] = sb;
                for (int j = 0; j <= T; ++j) {
                    const int d = s_dst[j], pos = s_pos[j];
                    if (d < 0 || pos >= ep.capacity) continue;
                    const int p = (j < T) ? m * T + j : M * T + m;
                    uint8_t* slab = ep.slab[d];
                    const size_t row = (size_t)ep.rank * ep.capacity + pos;
                    reinterpret_cast<uint2*>(slab + ep.L.recv_q + row * (K / 2))[kb] = make_uint2(lo, hi);
                    if (kb == 0) {
                        const int id = (j < T) ? topk_ids[p] : 0;
                        const int le = (j < T) ? id - (id / ep.e_local) * ep.e_local : ep.e_local;     // shared expert = local id E_local
                        const float w = (j < T) ? topk_w[p] : 1.0f;
                        reinterpret_cast<int4*>(slab + ep.L.recv_meta)[row] = make_int4(le, p, __float_as_int(w), 0);
                    }
                }
            }
            __syncthreads();
            // the chunk's block scales leave as 16-byte stores (K is a multiple of 256: 16 scales never straddle a chunk)
            const int parts = min((int)blockDim.x, bpr - kb0) / 16;
            for (int i = tid; i < (T + 1) * parts; i += blockDim.x) {
                const int j = i / parts, part = i - j * parts;
                const int d = s_dst[j], pos = s_pos[j];
                if (d < 0 || pos >= ep.capacity) continue;
                const size_t row = (size_t)ep.rank * ep.capacity + pos;
                reinterpret_cast<uint4*>(ep.slab[d] + ep.L.recv_sf + row * (K / 16) + kb0)[part] = reinterpret_cast<const uint4*>(s_sf)[part];
            }
            __syncthreads();
        }
    }
    // Last CTA to finish publishes the counts and the call flag on every peer.  The ticket orders memory at GPU scope
    // (release: this CTA's peer stores, seen through the barrier; acquire: the other CTAs'); the one system-scope release
    // is the flag store, cumulative over all of that and over the count stored just before it by the same thread.
    __syncthreads();
    if (tid == 0) s_last = (atom_acq_rel_add(&ep.state->ticket_dispatch, 1) == (int)gridDim.x - 1);
    __syncthreads();
    if (s_last && tid < ep.world) {
        const int d = tid;
        EpFlags* f = reinterpret_cast<EpFlags*>(ep.slab[d] + ep.L.flags);
        const int sent = s_total[d] + ((has_shared && d == ep.rank) ? M : 0);
        const int32_t call = ep.state->epoch + 1;
        const int32_t bad = (*(volatile int32_t*)status) != 0;
        f->dispatch_count[ep.rank] = min(sent, ep.capacity);
        st_release_sys(&f->dispatch_flag[ep.rank], call * 2 + bad);
    }
    if (s_last && tid == 0) ep.state->ticket_dispatch = 0;
    if (tid == 0) EP_MARK_MAX(ep, 22);
}

// ---------------------------------------------------------------------------------
// 3 gather + tables: wait (bounded) for every source's flag, make the dense list of the rows that arrived
// -- row i of the list is (source s, position i - src_base[s]), one single-expert "token" each -- and build
// the permutation tables over exactly those rows.  One CTA.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ int ep_source_of(const int32_t* base, int world, int i) {
    int s = 0;
    while (s + 1 < world && i >= base[s + 1]) ++s;
    return s;
}

__global__ void __launch_bounds__(TC_TILE_ROWS * 8)
ep_gather_tables_kernel(EpDev ep, TableArgs a, int smem_table_words) {
    extern __shared__ int32_t s_mem[];          // [E] counts, [3 * nthr] scan, then bitmap + running popcounts when they fit
    __shared__ int32_t s_base[EP_MAX_RANKS + 1];
    __shared__ int s_ok;
    const int tid = threadIdx.x, nthr = blockDim.x;
    int32_t* s_count = s_mem; int32_t* s_scan = s_mem + a.E;
    pdl_begin();
    if (tid == 0) EP_MARK_MIN(ep, 23);
    int32_t* status = a.ws.counters + CNT_STATUS;
    const EpFlags* f = reinterpret_cast<const EpFlags*>(ep.slab[ep.rank] + ep.L.flags);
    const int32_t call = ep.state->epoch + 1;
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < ep.world) {
        const int32_t v = wait_flag(&f->dispatch_flag[tid], call, ep.wait_ns);
        if (v < 0) { atomicExch(status, VMOE_ERR_TIMEOUT); s_ok = 0; }
        else if (v & 1) atomicCAS(status, 0, VMOE_ERR_PEER);          // the sender dropped rows: results are incomplete
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int s = 0; s < ep.world; ++s) {
            s_base[s] = run;
            run += s_ok ? min(max(f->dispatch_count[s], 0), ep.capacity) : 0;
        }
        s_base[ep.world] = run;
        for (int s = 0; s <= ep.world; ++s) ep.state->src_base[s] = s_base[s];
        ep.state->recv_rows = run;
    }
    __syncthreads();
    const int R = s_base[ep.world];
    const int4* meta = reinterpret_cast<const int4*>(ep.slab[ep.rank] + ep.L.recv_meta);
    a.M = R; a.words = (R + 31) / 32;
    // Everything a later phase of this CTA reads back lives in shared memory when it fits (ids, weights, expert
    // offsets, unit bases, slots, bitmap, running popcounts) and is copied out at the end; otherwise only the bitmap
    // and its popcounts do, or nothing does (the workspace holds room for all of it).
    int32_t* s_free = s_scan + 3 * nthr;
    const long long need_tables = 2LL * a.E * a.words, need_rest = 2LL * (a.E + 2) + 3LL * R;
    const bool shadow = need_tables + need_rest <= smem_table_words;
    int32_t* g_off = a.ws.expert_offsets; int32_t* g_ub = a.ws.tc_unit_base; int32_t* g_slot = a.ws.pair_slot;
    int32_t* ids = ep.flat_ids; float* wts = ep.flat_w;
    if (shadow) {
        a.ws.expert_offsets = s_free; a.ws.tc_unit_base = s_free + a.E + 2; a.ws.pair_slot = s_free + 2 * (a.E + 2);
        ids = a.ws.pair_slot + R; wts = reinterpret_cast<float*>(ids + R);
        s_free = ids + 2 * R;
        for (int i = tid; i < a.E + 2; i += nthr) a.ws.tc_unit_base[i] = 0;
    }
    if (shadow || need_tables <= smem_table_words) {
        a.ws.bitmap = reinterpret_cast<uint32_t*>(s_free);
        a.ws.word_prefix = reinterpret_cast<int32_t*>(a.ws.bitmap + (size_t)a.E * a.words);
    }
    for (int i = tid; i < R; i += nthr) {
        const int s = ep_source_of(s_base, ep.world, i);
        const int4 mt = meta[(size_t)s * ep.capacity + (i - s_base[s])];
        ids[i] = mt.x;
        wts[i] = __int_as_float(mt.z);
        if (shadow) { ep.flat_ids[i] = mt.x; ep.flat_w[i] = __int_as_float(mt.z); }     // the permutation of the rows reads them
    }
    a.ids = ids; a.w = wts;
    phase_clear(a, tid, nthr);
    __syncthreads();
    if (tid == 0) EP_MARK_MAX(ep, 24);
    phase_mark(a, tid, nthr);        __syncthreads();
    phase_count(a, tid >> 5, nthr >> 5, tid & 31, s_count); __syncthreads();
    phase_scan(a, tid, nthr, s_count, s_scan); __syncthreads();
    phase_place(a, tid, nthr);
    __syncthreads();
    if (shadow) {
        for (int i = tid; i < a.E + 2; i += nthr) g_off[i] = a.ws.expert_offsets[i];
        for (int i = tid; i < a.E + 1; i += nthr) g_ub[i] = a.ws.tc_unit_base[i];
        for (int i = tid; i < R; i += nthr) g_slot[i] = a.ws.pair_slot[i];
    }
    if (tid == 0) EP_MARK_MAX(ep, 25);
}

// ---------------------------------------------------------------------------------
// 4 permute: received FP4 rows -> sorted-slot order + scale atoms (B operand of the tensor-core GEMM), and
// the destination of each slot's output row in its owner's combine slab.  Grid-stride over the rows that
// arrived (their number is only known on the device).
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_permute_kernel(TcEpPermute e, int K, int tc_cap, Workspace ws) {
    pdl_begin();
    const int bpr = K / SF_BLOCK;
    const long long total = (long long)e.src_base[e.world] * bpr;
    constexpr int NB = 4;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long b0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; b0 < total; b0 += NB * stride) {
        long long bs[NB];
#pragma unroll
        for (int n = 0; n < NB; ++n) bs[n] = (b0 + n * stride < total) ? b0 + n * stride : -1;
        ep_permute_blocks<NB>(e, bs, K, tc_cap, ws);
    }
}

// 5b: the "rows are in place" flag when the token-major kernels ran (the weights-as-rows kernel publishes it itself)
__global__ void ep_signal_kernel(EpDev ep, const int32_t* status) {
    pdl_begin();                   // the down projection's peer stores are complete and visible to this grid
    if (threadIdx.x < ep.world) {
        EpFlags* f = reinterpret_cast<EpFlags*>(ep.slab[threadIdx.x] + ep.L.flags);
        const int32_t bad = (*(volatile const int32_t*)status) != 0;
        st_release_sys(&f->combine_flag[ep.rank], (ep.state->epoch + 1) * 2 + bad);
    }
}

// ---------------------------------------------------------------------------------
// 6 combine: out[m, :] = bf16( sum_{j < T} comb[m*T + j, :] + comb[M*T + m, :] ) (+ residual), fp32, ascending
// j: the same order as combine_kernel, over rows that arrived from the ranks owning the experts.  Nothing is
// written when a wait ran out or a rank marked its flag.  The last CTA advances the call counter.
// ---------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
ep_combine_kernel(EpDev ep, int M, int K, int T, int has_shared, const __nv_bfloat16* residual, __nv_bfloat16* out,
                  int32_t* status) {
    __shared__ int s_ok;
    pdl_begin();
    if (threadIdx.x == 0) EP_MARK_MIN(ep, 26);
    const EpFlags* f = reinterpret_cast<const EpFlags*>(ep.slab[ep.rank] + ep.L.flags);
    const int32_t call = ep.state->epoch + 1;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < ep.world) {
        const int32_t v = wait_flag(&f->combine_flag[threadIdx.x], call, ep.wait_ns);
        if (v < 0) { atomicExch(status, VMOE_ERR_TIMEOUT); s_ok = 0; }
        else if (v & 1) { atomicCAS(status, 0, VMOE_ERR_PEER); s_ok = 0; }
    }
    __syncthreads();
    if (s_ok && *(volatile int32_t*)status != 0) s_ok = 0;      // benign race: every thread stores the same value
    __syncthreads();
    if (s_ok) {
        const float* comb = reinterpret_cast<const float*>(ep.slab[ep.rank] + ep.L.comb);
        const int k4 = K / 4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)M * k4; i += (long long)gridDim.x * blockDim.x) {
            const int m = (int)(i / k4), c = (int)(i % k4);
            // all rows of the token are requested at once (the loop below would otherwise wait for each load in turn)
            float4 v[MAX_TOPK + 1];
#pragma unroll
            for (int j = 0; j <= MAX_TOPK; ++j) {
                const bool live = j < T || (j == MAX_TOPK && has_shared);
                const size_t row = j < T ? (size_t)(m * T + j) : (size_t)(M * T + m);
                v[j] = live ? __ldcg(reinterpret_cast<const float4*>(comb + row * K) + c) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int j = 0; j <= MAX_TOPK; ++j)        // ascending pair order, shared expert last
                if (j < T || (j == MAX_TOPK && has_shared)) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
            __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
            if (residual) {
                // x + moe(x) with the layer output rounded to bf16 first: the same bits as a separate bf16 add
                const uint2 r = reinterpret_cast<const uint2*>(residual + (size_t)m * K)[c];
                const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&r.x), r1 = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
                lo = __floats2bfloat162_rn(__bfloat162float(r0.x) + __bfloat162float(lo.x), __bfloat162float(r0.y) + __bfloat162float(lo.y));
                hi = __floats2bfloat162_rn(__bfloat162float(r1.x) + __bfloat162float(hi.x), __bfloat162float(r1.y) + __bfloat162float(hi.y));
            }
            uint2 o; o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(out + (size_t)m * K)[c] = o;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) EP_MARK_MAX(ep, 27);
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&ep.state->ticket_combine, 1) == (int)gridDim.x - 1) {
            ep.state->ticket_combine = 0;
            ep.state->epoch = call;           // every kernel of this call has read the old value
        }
    }
}

}  // namespace vmoe

using namespace vmoe;

// ---------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------
static int ep_check(const vmoe_ep_ctx* c) {
    if (!c) return VMOE_ERR_NULL;
    if (c->world < 1 || c->world > EP_MAX_RANKS || c->rank < 0 || c->rank >= c->world) return VMOE_ERR_SHAPE;
    if (c->experts_per_rank <= 0 || c->capacity <= 0 || c->max_local_tokens <= 0 || c->wait_limit_us < 0) return VMOE_ERR_SHAPE;
    for (int i = 0; i < c->world; ++i) if (!c->slab[i]) return VMOE_ERR_NULL;
    return VMOE_OK;
}

// the shape the local expert compute runs with: G * capacity single-expert "tokens", experts
// 0 .. E_local - 1 routed + id E_local = the shared expert
static vmoe_shape ep_local_shape(const vmoe_ep_ctx* c, const vmoe_shape* s, bool for_tables) {
    vmoe_shape l = *s;
    l.max_tokens = c->world * c->capacity;
    l.topk = 1;
    l.num_experts = c->experts_per_rank + (for_tables ? 1 : 0);
    l.num_global_experts = l.num_experts;
    l.has_shared = for_tables ? 0 : 1;
    l.path = VMOE_PATH_TC;
    return l;
}

// Entries of the tensor-core unit list of an expert-parallel workspace: the rows a rank receives depend on the
// other ranks' routing, so the list is sized for the worst case in 16-token units whatever this rank's own batch.
static int ep_tc_units(const vmoe_ep_ctx* c) {
    const long long rows = (long long)c->world * c->capacity;
    return (int)(c->experts_per_rank + 3 + rows / TC_UNIT_TOK_SMALL);
}

static size_t ep_extra_bytes(const vmoe_ep_ctx* c, const vmoe_shape* s) {
    const size_t rows = (size_t)c->world * c->capacity;
    const size_t P = (size_t)c->max_local_tokens * (s->topk + 1);
    // state, flat_ids, flat_w [rows], row_dst [rows], local topk ids / weights [P]
    return ep_align(sizeof(EpState)) + ep_align(rows * 4) * 2 + ep_align(rows * 8) + ep_align(P * 4) * 2;
}

extern "C" {

size_t vmoe_ep_slab_bytes(const vmoe_ep_ctx* ctx, const vmoe_shape* shape) {
    if (ep_check(ctx) || !shape) return 0;
    return ep_layout(ctx->world, ctx->capacity, ctx->max_local_tokens, shape->hidden, shape->topk).total;
}

size_t vmoe_ep_workspace_bytes(const vmoe_ep_ctx* ctx, const vmoe_shape* shape) {
    if (ep_check(ctx) || !shape) return 0;
    const vmoe_shape l = ep_local_shape(ctx, shape, true);
    vmoe_ws_layout L;
    if (compute_layout(&l, &L, ep_tc_units(ctx))) return 0;
    return L.total_bytes + ep_extra_bytes(ctx, shape);
}

int vmoe_ep_alloc(size_t bytes, void** out) {
    if (!out || bytes == 0) return VMOE_ERR_NULL;
    if (cudaMalloc(out, bytes) != cudaSuccess) return VMOE_ERR_CUDA;
    return cudaMemset(*out, 0, bytes) == cudaSuccess ? VMOE_OK : VMOE_ERR_CUDA;
}
int vmoe_ep_free(void* p) { return cuda_status(cudaFree(p)); }

int vmoe_ep_ipc_export(void* slab, void* handle_out_64_bytes) {
    if (!slab || !handle_out_64_bytes) return VMOE_ERR_NULL;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    return cuda_status(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out_64_bytes), slab));
}
int vmoe_ep_ipc_open(const void* handle_64_bytes, void** out) {
    if (!handle_64_bytes || !out) return VMOE_ERR_NULL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle_64_bytes, sizeof(h));
    return cuda_status(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
}
int vmoe_ep_ipc_close(void* p) { return cuda_status(cudaIpcCloseMemHandle(p)); }

int vmoe_ep_forward(const vmoe_ep_ctx* ctx, const vmoe_shape* shape, const vmoe_weights* routed,
                    const vmoe_weights* shared, const void* hidden_bf16, const float* router_logits,
                    const void* residual_bf16, void* out_bf16, int32_t M, void* workspace, size_t workspace_bytes,
                    void* stream) {
    int rc = ep_check(ctx);
    if (rc) return rc;
    if (!shape || !routed || !workspace) return VMOE_ERR_NULL;
    if (M > 0 && (!hidden_bf16 || !router_logits || !out_bf16)) return VMOE_ERR_NULL;   // a rank may bring no tokens
    if (shape->has_shared && !shared) return VMOE_ERR_NULL;
    if (M < 0 || M > ctx->max_local_tokens) return VMOE_ERR_SHAPE;
    if (shape->num_global_experts != ctx->world * ctx->experts_per_rank || shape->num_experts != ctx->experts_per_rank) return VMOE_ERR_SHAPE;
    if (shape->hidden % 256 || shape->inter % 256 || shape->topk < 1 || shape->topk > MAX_TOPK) return VMOE_ERR_SHAPE;
    if (!routed->w13_sf_atoms || !routed->w2_sf_atoms || (shape->has_shared && (!shared->w13_sf_atoms || !shared->w2_sf_atoms)))
        return VMOE_ERR_NULL;                              // the expert-parallel path runs on the tensor cores only
    if (workspace_bytes < vmoe_ep_workspace_bytes(ctx, shape)) return VMOE_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int K = shape->hidden, T = shape->topk;
    const vmoe_shape lt = ep_local_shape(ctx, shape, true), lk = ep_local_shape(ctx, shape, false);
    const int tc_units = ep_tc_units(ctx);
    Workspace ws;
    if ((rc = resolve_workspace(&lt, workspace, &ws, tc_units))) return rc;
    // EP scratch behind the regular workspace
    vmoe_ws_layout L;
    compute_layout(&lt, &L, tc_units);
    uint8_t* extra = static_cast<uint8_t*>(workspace) + L.total_bytes;
    const size_t rows = (size_t)ctx->world * ctx->capacity;
    const size_t P = (size_t)ctx->max_local_tokens * (T + 1);
    EpDev ep;
    memset(&ep, 0, sizeof(ep));
    ep.rank = ctx->rank; ep.world = ctx->world; ep.e_local = ctx->experts_per_rank; ep.capacity = ctx->capacity;
    ep.wait_ns = ctx->wait_limit_us > 0 ? (unsigned long long)ctx->wait_limit_us * 1000ull : MBAR_WAIT_LIMIT_NS;
    for (int i = 0; i < ctx->world; ++i) ep.slab[i] = static_cast<uint8_t*>(ctx->slab[i]);
    ep.L = ep_layout(ctx->world, ctx->capacity, ctx->max_local_tokens, K, T);
    ep.timeline = ws.timeline;
    auto take = [&](size_t b) { uint8_t* p = extra; extra += ep_align(b); return p; };
    ep.state = reinterpret_cast<EpState*>(take(sizeof(EpState)));
    ep.flat_ids = reinterpret_cast<int32_t*>(take(rows * 4));
    ep.flat_w = reinterpret_cast<float*>(take(rows * 4));
    ep.row_dst = reinterpret_cast<float**>(take(rows * 8));
    int32_t* loc_ids = reinterpret_cast<int32_t*>(take(P * 4));
    float* loc_w = reinterpret_cast<float*>(take(P * 4));
    int32_t* status = ws.counters + CNT_STATUS;
    const int has_shared = shape->has_shared ? 1 : 0;
    const int Eg = shape->num_global_experts;

    // 1 router
    if ((rc = launch_route(router_logits, M, Eg, T, loc_ids, loc_w, st))) return rc;
    {
        static bool attr_done = false;
        if (!attr_done) {
            cudaFuncSetAttribute(ep_gather_tables_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            attr_done = true;
        }
    }
    // 2 dispatch (+ plan): one CTA per local token; a rank without tokens still publishes its (empty) counts
    launch_pdl(ep_dispatch_kernel, (unsigned)(M > 0 ? M : 1), 256u, 0, st, static_cast<const __nv_bfloat16*>(hidden_bf16),
               loc_ids, loc_w, M, K, T, has_shared, ep, status);
    // Tokens per work unit and with them the kernel: chosen by the single-GPU rule (routed pairs per routed expert)
    // from the rows a rank receives under balanced routing, about its own M * T; any other row count is still
    // computed correctly, only not by the faster kernel.
    const int cap = tc_unit_cap(lk, M * T);
    // 3 gather + tables
    {
        TableArgs a;
        memset(&a, 0, sizeof(a));
        a.ids = ep.flat_ids; a.w = ep.flat_w; a.expert_map = nullptr;
        a.M = 0; a.T = 1; a.E = lt.num_experts; a.has_shared = 0; a.words = 0;
        a.num_global = lt.num_experts; a.tiles_d = 0; a.tc_cap = cap; a.gemv_units = 0;
        a.ws = ws;
        const unsigned nthr = TC_TILE_ROWS * 8;
        const size_t fixed = ((size_t)a.E + 3 * nthr) * sizeof(int32_t);
        const size_t smem = 200 * 1024;
        launch_pdl(ep_gather_tables_kernel, 1u, nthr, smem, st, ep, a, (int)((smem - fixed) / 4));
    }
    // 4 permute + 5 experts.  The weights-as-rows kernel permutes the received rows as its first work and publishes
    // the "rows are in place" flags from its last CTA; around the token-major kernels both are launches of their own.
    const WeightSet r{routed->w13, routed->w13_sf, routed->w13_gs, routed->w2, routed->w2_sf, routed->w2_gs};
    const WeightSet sh = shape->has_shared ? WeightSet{shared->w13, shared->w13_sf, shared->w13_gs, shared->w2, shared->w2_sf, shared->w2_gs}
                                           : r;
    PreparedSet prep{routed->w13_sf_atoms, routed->w2_sf_atoms,
                     shape->has_shared ? shared->w13_sf_atoms : routed->w13_sf_atoms,
                     shape->has_shared ? shared->w2_sf_atoms : routed->w2_sf_atoms};
    TcEpPermute perm;
    memset(&perm, 0, sizeof(perm));
    perm.recv_q = ep.slab[ctx->rank] + ep.L.recv_q; perm.recv_sf = ep.slab[ctx->rank] + ep.L.recv_sf;
    perm.recv_meta = reinterpret_cast<const int4*>(ep.slab[ctx->rank] + ep.L.recv_meta);
    for (int i = 0; i < ctx->world; ++i) perm.comb[i] = reinterpret_cast<float*>(ep.slab[i] + ep.L.comb);
    perm.src_base = ep.state->src_base; perm.flat_ids = ep.flat_ids; perm.row_dst = ep.row_dst;
    perm.world = ctx->world; perm.capacity = ctx->capacity;
    ws.row_dst = ep.row_dst;
    const int Mr = (int)rows;
    const bool in_kernel = cap == TC_UNIT_TOK_SMALL;
    if (in_kernel) {
        TcEpSignal sig;
        memset(&sig, 0, sizeof(sig));
        for (int i = 0; i < ctx->world; ++i)
            sig.flag[i] = &reinterpret_cast<EpFlags*>(ep.slab[i] + ep.L.flags)->combine_flag[ctx->rank];
        sig.world = ctx->world; sig.epoch = &ep.state->epoch; sig.ticket = &ep.state->ticket_experts;
        if ((rc = launch_tc(lk, r, sh, prep, Mr, ws, st, TC_PHASE_GATE_UP | TC_PHASE_DOWN, nullptr, nullptr, nullptr, cap, Mr, &sig,
                            nullptr, nullptr, &perm))) return rc;
    } else {
        launch_pdl(ep_permute_kernel, (unsigned)(2 * 148), 256u, 0, st, perm, K, cap, ws);
        if ((rc = launch_tc(lk, r, sh, prep, Mr, ws, st, TC_PHASE_GATE_UP | TC_PHASE_DOWN, nullptr, nullptr, nullptr, cap, Mr))) return rc;
        launch_pdl(ep_signal_kernel, 1u, 32u, 0, st, ep, static_cast<const int32_t*>(status));
    }
    // 6 combine
    // one output element (four columns) per thread, like the single-GPU combine; at least one CTA (a rank without
    // tokens still waits for the flags and advances the call counter)
    const long long cn = (long long)M * (K / 4);
    const unsigned cgrid = (unsigned)(cn > 0 ? (cn + 255) / 256 < 65535 ? (cn + 255) / 256 : 65535 : 1);
    launch_pdl(ep_combine_kernel, cgrid, 256u, 0, st, ep, M, K, T, has_shared, static_cast<const __nv_bfloat16*>(residual_bf16),
               static_cast<__nv_bfloat16*>(out_bf16), status);
    return cuda_status(cudaGetLastError());
}

int vmoe_ep_read_status(const vmoe_ep_ctx* ctx, const vmoe_shape* shape, void* workspace, void* stream) {
    int rc = ep_check(ctx);
    if (rc) return rc;
    if (!shape || !workspace) return VMOE_ERR_NULL;
    const vmoe_shape lt = ep_local_shape(ctx, shape, true);
    Workspace ws;
    if ((rc = resolve_workspace(&lt, workspace, &ws, ep_tc_units(ctx)))) return rc;
    int32_t v = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemcpyAsync(&v, ws.counters + CNT_STATUS, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return VMOE_ERR_CUDA;
    if (cudaStreamSynchronize(st) != cudaSuccess) return VMOE_ERR_CUDA;
    if (v != 0) cudaMemsetAsync(ws.counters + CNT_STATUS, 0, 4, st);
    return v;
}

}  // extern "C"
