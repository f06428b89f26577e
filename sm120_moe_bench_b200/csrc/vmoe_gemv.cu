// Decode path: bandwidth-bound streaming GEMV kernels over NVFP4 expert weights.
//
//   gate_up_kernel : GEMM1 (a8) + x alpha1 + SwiGLU + FP4 re-quantisation (a9)
//   down_kernel    : GEMM2 (a10) + (router weight x alpha2) scaling into per-slot fp32 rows
//
// Math follows fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:323-538 of the reference;
// the structure does not.  Each distinct expert is read ONCE for all tokens routed to it (work
// units of <= 4 tokens from the permutation tables).  Persistent CTAs pull (unit, row tile)
// items from a device-side queue; a producer warp streams E2M1 rows and E4M3 scale rows into a
// shared-memory ring with the bulk-copy (TMA) engine and mbarriers; four consumer warps read the
// ring with 128-bit loads, turn packed E2M1 into f16x2 with cvt, form the exact per-16-block
// products sums with HFMA2 (8 products of <= 36 in steps of 0.25 per half: exact in f16), scale
// them in fp32 and reduce across lanes with shuffles.
#include "vmoe_common.cuh"

#include <mutex>
#include <vector>

namespace vmoe {

constexpr int CONSUMER_WARPS = 4;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int GEMV_THREADS = CONSUMERS + 32;      // + one producer warp
constexpr int ROWS_PER_THREAD = 8;                // rows a thread covers per stage
constexpr int RING = 3;                           // stages in flight per CTA
constexpr int GATE_UP_TILE = 16;                  // n per gate_up item (16 gate rows + 16 up rows)
constexpr int DOWN_TILE = 32;                     // output rows per down item

struct GemvParams {
    WeightSet routed, shared;
    Workspace ws;
    int K, N, E, tiles;          // tiles = items per unit
    int row_bytes, sf_row_bytes; // one weight row / one scale row
    int stage_rows;              // rows per stage (8 gate_up, 32 down)
    int stage_bytes;
};

struct __align__(16) StageInfo { int expert, slot0, ntok_stage, tile; };

__device__ __forceinline__ void named_barrier_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---------------------------------------------------------------------------------
// Per-thread activation fragment of one token: 32 consecutive elements (2 blocks).
// ---------------------------------------------------------------------------------
struct ActFrag { __half2 v[16]; float s0, s1; };

__device__ __forceinline__ void load_act(ActFrag& a, const uint8_t* q, const uint8_t* sf, bool valid) {
    if (valid) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 16; ++i) a.v[i] = cvt_e2m1x2((w[i >> 2] >> (8 * (i & 3))) & 0xFF);
        const __half2 s = cvt_e4m3x2(__ldg(reinterpret_cast<const uint16_t*>(sf)));
        a.s0 = __low2float(s); a.s1 = __high2float(s);
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) a.v[i] = __float2half2_rn(0.f);
        a.s0 = 0.f; a.s1 = 0.f;
    }
}

// 8 rows x T tokens partial dot products of this thread's 32-element chunk.
template <int T>
__device__ __forceinline__ void stage_dot(const uint8_t* __restrict__ wrow, const uint8_t* __restrict__ sfrow,
                                          int row_bytes, int sf_row_bytes, const ActFrag (&act)[T],
                                          float (&acc)[ROWS_PER_THREAD][T]) {
#pragma unroll
    for (int r = 0; r < ROWS_PER_THREAD; ++r) {
        const uint4 raw = *reinterpret_cast<const uint4*>(wrow + r * row_bytes);
        const __half2 s = cvt_e4m3x2(*reinterpret_cast<const uint16_t*>(sfrow + r * sf_row_bytes));
        const float ws0 = __low2float(s), ws1 = __high2float(s);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        __half2 wv[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) wv[i] = cvt_e2m1x2((w[i >> 2] >> (8 * (i & 3))) & 0xFF);
#pragma unroll
        for (int t = 0; t < T; ++t) {
            __half2 a0 = __float2half2_rn(0.f), a1 = a0;
#pragma unroll
            for (int i = 0; i < 8; ++i) a0 = __hfma2(wv[i], act[t].v[i], a0);
#pragma unroll
            for (int i = 8; i < 16; ++i) a1 = __hfma2(wv[i], act[t].v[i], a1);
            const float f0 = __low2float(a0) + __high2float(a0);
            const float f1 = __low2float(a1) + __high2float(a1);
            acc[r][t] = fmaf(f0, ws0 * act[t].s0, fmaf(f1, ws1 * act[t].s1, 0.f));
        }
    }
}

// Transposed butterfly: 8 per-lane partials -> the lane group (lane >> 2) holds the warp total
// of row ((lane>>4)&1)*4 + ((lane>>3)&1)*2 + ((lane>>2)&1) in every one of its 4 lanes.
__device__ __forceinline__ float warp_reduce8(const float (&v)[8], int lane) {
    float a[4], b[2], c;
    const bool h4 = lane & 16, h3 = lane & 8, h2 = lane & 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = h4 ? v[i] : v[i + 4];
        const float keep = h4 ? v[i + 4] : v[i];
        a[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = h3 ? a[i] : a[i + 2];
        const float keep = h3 ? a[i + 2] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    {
        const float send = h2 ? b[0] : b[1];
        const float keep = h2 ? b[1] : b[0];
        c = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    return c;
}
__device__ __forceinline__ int reduce8_row(int lane) { return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1); }

// ---------------------------------------------------------------------------------
// Shared-memory layout
// ---------------------------------------------------------------------------------
struct RingState {
    uint64_t full[RING];
    uint64_t empty[RING];
    StageInfo info[RING];
};

__device__ __forceinline__ void report_timeout(const Workspace& ws) { atomicExch(&ws.counters[CNT_STATUS], VMOE_ERR_TIMEOUT); }

// Producer: one lane.  MODE 0 = gate_up (4 stages per item), MODE 1 = down (1 stage per item).
template <int MODE>
__device__ void producer_loop(const GemvParams& p, RingState* rs, uint8_t* ring, int queue_idx) {
    const int num_units = p.ws.counters[CNT_UNITS];
    const long long total = (long long)num_units * p.tiles;
    uint32_t g = 0;
    bool ok = true;
    auto acquire = [&](int& slot) -> bool {
        slot = g % RING;
        if (g >= RING && !mbar_wait(&rs->empty[slot], ((g / RING) - 1) & 1)) return false;
        return true;
    };
    while (ok) {
        const long long item = atomicAdd(&p.ws.counters[queue_idx], 1);
        if (item >= total) break;
        const int unit = (int)(item / p.tiles), tile = (int)(item % p.tiles);
        const int4 u = p.ws.units[unit];
        const bool sh = (u.x >= p.E);
        const WeightSet& W = sh ? p.shared : p.routed;
        const int e = sh ? 0 : u.x;
        constexpr int NST = (MODE == 0) ? 4 : 1;
#pragma unroll 1
        for (int s = 0; s < NST; ++s) {
            int slot;
            if (!acquire(slot)) { ok = false; break; }
            long long row;
            const uint8_t *wb, *sb;
            if (MODE == 0) {
                row = (long long)e * 2 * p.N + (s >= 2 ? p.N : 0) + tile * GATE_UP_TILE + (s & 1) * 8;
                wb = W.w13; sb = W.w13_sf;
            } else {
                row = (long long)e * p.K + (long long)tile * DOWN_TILE;
                wb = W.w2; sb = W.w2_sf;
            }
            rs->info[slot] = StageInfo{u.x, u.y, u.z | (s << 8), tile};
            uint8_t* dst = ring + (size_t)slot * p.stage_bytes;
            const uint32_t wbytes = p.stage_rows * p.row_bytes, sbytes = p.stage_rows * p.sf_row_bytes;
            mbar_arrive_expect_tx(&rs->full[slot], wbytes + sbytes);
            bulk_g2s(dst, wb + row * p.row_bytes, wbytes, &rs->full[slot]);
            bulk_g2s(dst + wbytes, sb + row * p.sf_row_bytes, sbytes, &rs->full[slot]);
            ++g;
        }
    }
    // end marker (also sent after a timeout so that consumers leave)
    int slot;
    if (!ok) report_timeout(p.ws);
    if (acquire(slot)) {
        rs->info[slot] = StageInfo{-1, 0, 0, 0};
        mbar_arrive(&rs->full[slot]);
    } else {
        report_timeout(p.ws);
    }
}

// ---------------------------------------------------------------------------------
// gate_up consumer: one item = 4 stages (gate 0-7, gate 8-15, up 0-7, up 8-15 of a 16-n tile)
// ---------------------------------------------------------------------------------
template <int T>
__device__ __forceinline__ bool gate_up_item(const GemvParams& p, RingState* rs, const uint8_t* ring,
                                             float* red, uint32_t& g, StageInfo inf, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int ntok = inf.ntok_stage & 0xFF;
    const bool cvalid = tid * 32 < p.K;
    ActFrag act[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
        const bool v = cvalid && t < ntok;
        const int tok = v ? p.ws.gather_idx[inf.slot0 + t] : 0;
        load_act(act[t], p.ws.act_q + (size_t)tok * (p.K / 2) + tid * 16,
                 p.ws.act_sf + (size_t)tok * (p.K / 16) + tid * 2, v);
    }
#pragma unroll 1
    for (int s = 0; s < 4; ++s) {
        const int slot = g % RING;
        if (s > 0) {
            if (!mbar_wait(&rs->full[slot], (g / RING) & 1)) { report_timeout(p.ws); return false; }
        }
        const uint8_t* st = ring + (size_t)slot * p.stage_bytes;
        float acc[ROWS_PER_THREAD][T];
        if (cvalid) {
            stage_dot<T>(st + tid * 16, st + p.stage_rows * p.row_bytes + tid * 2, p.row_bytes, p.sf_row_bytes, act, acc);
        } else {
#pragma unroll
            for (int r = 0; r < ROWS_PER_THREAD; ++r)
#pragma unroll
                for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&rs->empty[slot]);
        ++g;
#pragma unroll
        for (int t = 0; t < T; ++t) {
            float v[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) v[r] = acc[r][t];
            const float tot = warp_reduce8(v, lane);
            if ((lane & 3) == 0) red[((s * CONSUMER_WARPS + warp) * 8 + reduce8_row(lane)) * TOK_PER_UNIT + t] = tot;
        }
    }
    named_barrier_sync(1, CONSUMERS);
    // epilogue: 16 threads per token
    if (tid < 16 * T) {
        const unsigned mask = (T == 1) ? 0x0000ffffu : 0xffffffffu;
        const int n = tid & 15, t = tid >> 4;
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int w = 0; w < CONSUMER_WARPS; ++w) {
            gate += red[(((n >> 3) * CONSUMER_WARPS + w) * 8 + (n & 7)) * TOK_PER_UNIT + t];
            up   += red[(((2 + (n >> 3)) * CONSUMER_WARPS + w) * 8 + (n & 7)) * TOK_PER_UNIT + t];
        }
        const bool sh = inf.expert >= p.E;
        const float alpha1 = sh ? p.shared.w13_gs[0] : p.routed.w13_gs[inf.expert];
        gate *= alpha1; up *= alpha1;
        const float sw = up * silu(gate);
        float gm = fabsf(sw);
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) gm = fmaxf(gm, __shfl_xor_sync(mask, gm, o));
        const uint8_t sb = e4m3_encode(fmaxf(gm / 6.0f, 1e-30f));
        float sc = e4m3_decode(sb);
        if (sc < 1e-30f) sc = 1e-30f;
        const uint32_t nib = e2m1_encode(ScaleDivider(sc)(sw));
        const uint32_t nb = __shfl_down_sync(mask, nib, 1);
        if (t < ntok) {
            const size_t slot_row = (size_t)(inf.slot0 + t);
            if ((n & 1) == 0) p.ws.inter_q[slot_row * (p.N / 2) + (inf.tile * GATE_UP_TILE + n) / 2] = (uint8_t)(nib | (nb << 4));
            if (n == 0) p.ws.inter_sf[slot_row * (p.N / 16) + inf.tile] = sb;
        }
    }
    return true;
}

__global__ void __launch_bounds__(GEMV_THREADS)
gate_up_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    RingState* rs = reinterpret_cast<RingState*>(smem + (size_t)RING * p.stage_bytes);
    float* red_base = reinterpret_cast<float*>(rs + 1);   // [2][4 stages][4 warps][8 rows][4 tok]
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < RING; ++i) { mbar_init(&rs->full[i], 1); mbar_init(&rs->empty[i], CONSUMER_WARPS); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();
    if (tid >= CONSUMERS) {
        if (tid == CONSUMERS) producer_loop<0>(p, rs, ring, CNT_QUEUE1);
        return;
    }
    uint32_t g = 0; int parity = 0;
    while (true) {
        const int slot = g % RING;
        if (!mbar_wait(&rs->full[slot], (g / RING) & 1)) { report_timeout(p.ws); break; }
        const StageInfo inf = rs->info[slot];
        if (inf.expert < 0) break;
        float* red = red_base + parity * (4 * CONSUMER_WARPS * 8 * TOK_PER_UNIT);
        const int ntok = inf.ntok_stage & 0xFF;
        bool ok;
        if (ntok == 1)      ok = gate_up_item<1>(p, rs, ring, red, g, inf, tid);
        else if (ntok == 2) ok = gate_up_item<2>(p, rs, ring, red, g, inf, tid);
        else                ok = gate_up_item<4>(p, rs, ring, red, g, inf, tid);
        if (!ok) break;
        parity ^= 1;
    }
}

// ---------------------------------------------------------------------------------
// down consumer: one item = one stage of 32 output rows; warp w takes rows 8w..8w+7,
// lane = 32-element chunk of the intermediate.
// ---------------------------------------------------------------------------------
template <int T>
__device__ __forceinline__ void down_item(const GemvParams& p, const uint8_t* st, StageInfo inf, int tid) {
    const int lane = tid & 31, warp = tid >> 5;
    const int ntok = inf.ntok_stage & 0xFF;
    const bool cvalid = lane * 32 < p.N;
    ActFrag act[T];
#pragma unroll
    for (int t = 0; t < T; ++t) {
        const bool v = cvalid && t < ntok;
        const size_t row = v ? (size_t)(inf.slot0 + t) : 0;
        load_act(act[t], p.ws.inter_q + row * (p.N / 2) + lane * 16, p.ws.inter_sf + row * (p.N / 16) + lane * 2, v);
    }
    float acc[ROWS_PER_THREAD][T];
    if (cvalid) {
        stage_dot<T>(st + (size_t)warp * 8 * p.row_bytes + lane * 16,
                     st + p.stage_rows * p.row_bytes + (size_t)warp * 8 * p.sf_row_bytes + lane * 2,
                     p.row_bytes, p.sf_row_bytes, act, acc);
    } else {
#pragma unroll
        for (int r = 0; r < ROWS_PER_THREAD; ++r)
#pragma unroll
            for (int t = 0; t < T; ++t) acc[r][t] = 0.f;
    }
    const bool sh = inf.expert >= p.E;
    const float alpha2 = sh ? p.shared.w2_gs[0] : p.routed.w2_gs[inf.expert];
    const int j = inf.tile * DOWN_TILE + warp * 8 + reduce8_row(lane);
#pragma unroll
    for (int t = 0; t < T; ++t) {
        float v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) v[r] = acc[r][t];
        const float tot = warp_reduce8(v, lane);
        if ((lane & 3) == 0 && t < ntok) {
            const int slot_row = inf.slot0 + t;
            const float scale = p.ws.scatter_weights[slot_row] * alpha2;
            p.ws.pair_out[(size_t)slot_row * p.K + j] = scale * tot;
        }
    }
}

__global__ void __launch_bounds__(GEMV_THREADS)
down_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    RingState* rs = reinterpret_cast<RingState*>(smem + (size_t)RING * p.stage_bytes);
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < RING; ++i) { mbar_init(&rs->full[i], 1); mbar_init(&rs->empty[i], CONSUMER_WARPS); }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();
    if (tid >= CONSUMERS) {
        if (tid == CONSUMERS) producer_loop<1>(p, rs, ring, CNT_QUEUE2);
        return;
    }
    uint32_t g = 0;
    while (true) {
        const int slot = g % RING;
        if (!mbar_wait(&rs->full[slot], (g / RING) & 1)) { report_timeout(p.ws); break; }
        const StageInfo inf = rs->info[slot];
        if (inf.expert < 0) break;
        const uint8_t* st = ring + (size_t)slot * p.stage_bytes;
        const int ntok = inf.ntok_stage & 0xFF;
        if (ntok == 1)      down_item<1>(p, st, inf, tid);
        else if (ntok == 2) down_item<2>(p, st, inf, tid);
        else                down_item<4>(p, st, inf, tid);
        __syncwarp();
        if ((tid & 31) == 0) mbar_arrive(&rs->empty[slot]);
        ++g;
    }
}

// ---------------------------------------------------------------------------------
// Launchers
// ---------------------------------------------------------------------------------
static int g_sm_count = 0;
static int sm_count() {
    if (g_sm_count == 0) {
        int dev = 0; cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    return g_sm_count;
}

static size_t gemv_smem(const GemvParams& p, bool gate_up) {
    size_t b = (size_t)RING * p.stage_bytes + sizeof(RingState);
    if (gate_up) b += 2 * 4 * CONSUMER_WARPS * 8 * TOK_PER_UNIT * sizeof(float);
    return b + 128;
}

static void fill(GemvParams& p, const vmoe_shape& s, const WeightSet& r, const WeightSet& sh, const Workspace& ws) {
    p.routed = r; p.shared = sh; p.ws = ws; p.K = s.hidden; p.N = s.inter; p.E = s.num_experts;
}

template <typename Kern>
static int launch_persistent(Kern kern, const GemvParams& p, size_t smem, int M, int units_hint, cudaStream_t st) {
    // attribute + occupancy are looked up once per (kernel, device, smem size)
    struct Cached { const void* kern; int dev; size_t smem; int per_sm; };
    static std::mutex mu;
    static std::vector<Cached> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (const Cached& c : cache)
            if (c.kern == (const void*)kern && c.dev == dev && c.smem == smem) per_sm = c.per_sm;
        if (per_sm == 0) {
            if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return VMOE_ERR_CUDA;
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, GEMV_THREADS, smem);
            if (per_sm < 1) per_sm = 1;
            cache.push_back(Cached{(const void*)kern, dev, smem, per_sm});
        }
    }
    long long want = (long long)units_hint * p.tiles;          // upper bound on items
    long long grid = (long long)sm_count() * per_sm;
    if (want < grid) grid = want;
    if (grid < 1) grid = 1;
    (void)M;
    kern<<<(unsigned)grid, GEMV_THREADS, smem, st>>>(p);
    return cuda_status(cudaGetLastError());
}

int launch_gate_up(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, int M,
                   const Workspace& ws, cudaStream_t st) {
    if (M == 0) return VMOE_OK;
    GemvParams p; fill(p, s, routed, shared, ws);
    p.tiles = s.inter / GATE_UP_TILE;
    p.row_bytes = s.hidden / 2; p.sf_row_bytes = s.hidden / 16;
    p.stage_rows = 8; p.stage_bytes = p.stage_rows * (p.row_bytes + p.sf_row_bytes);
    const int units_hint = min(M * s.topk + (s.has_shared ? M : 0), max_units(&s));
    return launch_persistent(gate_up_kernel, p, gemv_smem(p, true), M, units_hint, st);
}

int launch_down(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, int M,
                const Workspace& ws, cudaStream_t st) {
    if (M == 0) return VMOE_OK;
    GemvParams p; fill(p, s, routed, shared, ws);
    p.tiles = s.hidden / DOWN_TILE;
    p.row_bytes = s.inter / 2; p.sf_row_bytes = s.inter / 16;
    p.stage_rows = DOWN_TILE; p.stage_bytes = p.stage_rows * (p.row_bytes + p.sf_row_bytes);
    const int units_hint = min(M * s.topk + (s.has_shared ? M : 0), max_units(&s));
    return launch_persistent(down_kernel, p, gemv_smem(p, false), M, units_hint, st);
}

}  // namespace vmoe
