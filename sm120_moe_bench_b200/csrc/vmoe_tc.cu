// Tensor-core path for memory-bound batches: block-scaled tcgen05.mma (kind::mxf4nvf4, 16-element E4M3
// scales) with the operand roles swapped, gate_up and down projection in ONE persistent kernel.
//
// The 128 rows of the UMMA tile are WEIGHT rows (A operand, streamed once from HBM by TMA with the 128-byte
// swizzle), the N dimension (8 or 16) holds the tokens routed to the expert (B operand, rows of the slot-
// ordered activation matrix).  With few tokens per expert this is a tensor-core GEMV: the FP4 decode happens
// inside the tensor core instead of on the conversion (XU) pipe, which a CUDA-core GEMV saturates long before
// HBM does.
//
// Work of one launch:
//   first, on the epilogue warps: the permuting activation quantiser (a6) -- chunks of 256 sixteen-element blocks,
//     chunk c on CTA c mod gridDim.x -- while the producers already stream the first weight tiles; a producer waits
//     (bounded) for the count of finished chunks before its first token-tile copy;
//   gate_up item (unit u, row tile t): 128 gate rows + the matching 128 up rows of the unit's expert over all
//     of K; epilogue = x alpha1, SiLU * up, FP4 re-quantisation of the intermediate (a8 + a9), then one
//     release-increment of unit_done[u] per epilogue warp;
//   down item (unit u, row tile t): 128 rows of w2 over all of N; its producer first streams the weight tiles
//     into the ring, then makes sure (bounded wait; normally seen complete one item earlier) that all gate_up
//     tiles of unit u are done before it loads the intermediate; epilogue = x (router weight x alpha2) -> fp32
//     row segment (a10), then -- smallest batches of the single-GPU forward -- one increment of
//     token_done[token, t] per token of the unit; whoever completes a token's count sums that token's rows for
//     these 128 columns in the fixed pair order and writes bf16 (a11).
// All gate_up items precede all down items in the queue and a gate_up item never waits, so a down item only
// ever waits for items that running CTAs already hold: no grid barrier, and the tail of one projection overlaps
// the head of the next.  The first item of a CTA is its block index and the quantiser chunks are assigned by block
// index too, so -- like any grid sized to the SM count -- the launch assumes that every CTA gets an SM; if a
// foreign kernel keeps one away for longer than the wait limit the call ends with VMOE_ERR_TIMEOUT, never in a
// hang.  Used alone (stage entry points) a phase mask selects one kind of item and nothing waits.
//
// Math follows fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:323-563 of the reference; its structure
// (one cooperative kernel, four grid barriers, partial sums per K group) is not reproduced.
// Warp roles per persistent CTA: warp 0 = TMA / bulk-copy producer, warp 1 = MMA issuer and TMEM owner,
// warps 2-9 = epilogue: two sets of four warps (one TMEM lane quadrant each) take the items in turn, so that the
// publish latency of one item (stores -> release -> counter) hides under the next item.  Every wait is bounded.
#include "vmoe_tc_common.cuh"
#include "vmoe_phases.cuh"

#include <string.h>

#include <mutex>
#include <unordered_map>

#include <cuda.h>
#include <cudaTypedefs.h>

namespace vmoe {

// One ring stage serves either kind of item:
//   gate_up: A0 = gate tile, A1 = up tile of one 256-element k-block; one token tile; 2 + 1 scale tiles
//   down:    A0, A1 = two consecutive k-blocks of the same 128 rows; two token tiles; 2 + 2 scale tiles
constexpr int FU_UT = TC_UNIT_TOK_SMALL;               // tokens per unit (UMMA N <= 16)
constexpr int FU_B_TILE = FU_UT * TC_KB_BYTES;          // 2 KiB
constexpr int FU_OFF_A1 = TC_A_TILE;
constexpr int FU_OFF_SFA = 2 * TC_A_TILE;               // [2][4 atoms]
constexpr int FU_OFF_B = FU_OFF_SFA + 2 * TC_SF_TILE;   // [2][16 x 128]
constexpr int FU_OFF_SFB = FU_OFF_B + 2 * FU_B_TILE;    // [2][4 atoms]
constexpr int FU_STAGE_BYTES = FU_OFF_SFB + 2 * TC_SF_TILE;     // 45056
constexpr int FU_STAGES = TC_SMEM_BUDGET / FU_STAGE_BYTES;      // 5
constexpr int FU_ACC_STRIDE = 2 * FU_UT;                // TMEM columns per accumulator buffer (gate | up)
constexpr int FU_NBUF = 4;
constexpr int FU_SF_COLS = 64;                          // scale columns of one stage: A tiles at +0, +16; B tiles at +32, +48
static_assert(FU_STAGES >= 3 && FU_STAGES <= 12, "ring depth");
static_assert(FU_NBUF * FU_ACC_STRIDE <= TC_SF_COL0 && TC_SF_COL0 + 2 * FU_SF_COLS <= TC_TMEM_COLS, "TMEM columns");

struct FuParams {
    CUtensorMap map_w13_routed, map_w13_shared;   // [rows, K/2] bytes, box 128 x 128, swizzle 128B
    CUtensorMap map_w2_routed, map_w2_shared;
    CUtensorMap map_act[2], map_inter[2];          // [slots, K/2] bytes, box 128 x {8, 16}
    const uint8_t* sfa13_routed; const uint8_t* sfa13_shared;     // scale atoms [rows/128][K/64][512]
    const uint8_t* sfa2_routed;  const uint8_t* sfa2_shared;
    const float* gs13_routed; const float* gs13_shared; const float* gs2_routed; const float* gs2_shared;
    Workspace ws;
    int hidden, N, E;
    int tiles_g, tiles_d;      // row tiles per unit: N / 128, hidden / 128
    int ks_d;                  // k-blocks per stage of a down item (2 when N / 256 is even)
    int phases;
    int queue;                 // counter index of the work queue
    // combine inside the kernel (single-GPU forward); out == NULL: rows only
    __nv_bfloat16* out; const __nv_bfloat16* residual;
    int T, has_shared, M;
    // permuting activation quantiser as the kernel's first work (pq_blocks = M * K / 16; 0 = done by the caller)
    int pq_blocks, tc_cap;
    TcQuant quant;
    int has_ep_permute;        // expert parallelism: the first work is the permutation of the received rows instead
    TcEpPermute ep_permute;
    int has_signal;
    TcEpSignal signal;
};

__device__ __forceinline__ int32_t ld_acquire_gpu(const int32_t* p) {
    int32_t v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// Bounded wait for *p >= want (another CTA's release-increments); false when the limit passes.
__device__ __forceinline__ bool wait_counter(const int32_t* p, int32_t want) {
    if (ld_acquire_gpu(p) >= want) return true;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t i = 1;; ++i) {
        if (ld_acquire_gpu(p) >= want) return true;
        if ((i & 15u) == 0 && global_timer_ns() - t0 > MBAR_WAIT_LIMIT_NS) return false;
    }
}

constexpr int FU_EPI_SETS = 2;                          // two sets of four epilogue warps take the items in turn
constexpr int FU_THREADS = 64 + FU_EPI_SETS * 128;      // producer warp, MMA warp, epilogue warps

struct FuShared {
    uint64_t full[FU_STAGES], empty[FU_STAGES];
    uint64_t tmem_full[FU_NBUF], tmem_empty[FU_NBUF];
    uint64_t epi_bar[FU_EPI_SETS];    // rendezvous of the four warps of an epilogue set (down items with the combine)
    TcStageInfo info[FU_STAGES];
    TcStageInfo epi[FU_NBUF];
    uint32_t tmem_base;
    int abort_flag;
    int last_cta;
};
constexpr int FU_PQ_CHUNK = FU_EPI_SETS * 128;          // 16-element blocks per chunk: one per epilogue thread

__device__ __forceinline__ void fu_timeout(const Workspace& ws, FuShared* sh) {
    atomicExch(&ws.counters[CNT_STATUS], VMOE_ERR_TIMEOUT);
    atomicExch(&sh->abort_flag, 1);
}
// kind of a stage record: TcStageInfo::pad[0]; k-blocks per stage: pad[1]
enum { ITEM_GATE_UP = 0, ITEM_DOWN = 1 };

struct FuItem { int kind, unit, tile; };

// ---------------------------------------------------------------------------------
// producer: the stages of one item.  NA = weight matrices per item (2: gate + up, 1: down), KS = k-blocks per
// stage.  Warp-uniform; one elected lane issues the copies.  Returns false when a wait ran out.
// ---------------------------------------------------------------------------------
template <int NA, int KS>
__device__ __forceinline__ bool fu_produce_item(const FuParams& p, uint8_t* smem, FuShared* sh, bool leader, uint32_t& g,
                                                const FuItem& it, const int4& u, float alpha, bool wait_unit, bool& wait_quant) {
    constexpr bool DOWN = NA == 1;
    const bool shd = u.x >= p.E;
    const int e = shd ? 0 : u.x;
    const int nbox = u.w;
    const CUtensorMap* ma = DOWN ? (shd ? &p.map_w2_shared : &p.map_w2_routed) : (shd ? &p.map_w13_shared : &p.map_w13_routed);
    const uint8_t* sfa = DOWN ? (shd ? p.sfa2_shared : p.sfa2_routed) : (shd ? p.sfa13_shared : p.sfa13_routed);
    const CUtensorMap* mb = DOWN ? &p.map_inter[nbox == 8 ? 0 : 1] : &p.map_act[nbox == 8 ? 0 : 1];
    const uint8_t* sfb = DOWN ? p.ws.inter_sf_atoms : p.ws.act_sf_atoms;
    const int K = DOWN ? p.N : p.hidden;                 // reduction length
    const int rows = DOWN ? p.hidden : 2 * p.N;          // weight rows per expert
    const int steps = (K / 256) / KS;
    const uint32_t bytes = NA * KS * (TC_A_TILE + TC_SF_TILE) + KS * (nbox * TC_KB_BYTES + TC_SF_TILE);
    for (int s = 0; s < steps; ++s) {
        const int slot = g % FU_STAGES;
        bool w = true;
        if (g >= (uint32_t)FU_STAGES) w = mbar_wait(&sh->empty[slot], ((g / FU_STAGES) - 1) & 1);
        w = w && !(*(volatile int*)&sh->abort_flag);
        if (!__all_sync(0xffffffffu, w)) return false;
        uint8_t* st = smem + (size_t)slot * FU_STAGE_BYTES;
        const int kb0 = s * KS;                       // first k-block of this stage
        if (leader) {
            sh->info[slot] = TcStageInfo{u.x, u.y, u.z, nbox, it.tile, it.unit, s, s == steps - 1, s == steps - 1 ? alpha : 0.f, {it.kind, KS, 0}};
            mbar_arrive_expect_tx(&sh->full[slot], bytes);
        }
        // weights and their scale atoms (the atoms of consecutive k-blocks of one row tile are contiguous)
#pragma unroll
        for (int a = 0; a < NA; ++a) {
            // gate_up: A0 = rows [tile*128, +128) of the gate half, A1 = the same rows of the up half
            const long long row = (long long)e * rows + (NA == 2 ? a * p.N : 0) + it.tile * TC_ROWS;
            const uint8_t* sfa_src = sfa + ((size_t)(row / TC_ROWS) * (K / 64) + (size_t)kb0 * 4) * 512;
#pragma unroll
            for (int kk = 0; kk < KS; ++kk)
                if (leader) tma_load_2d(st + (a * KS + kk) * TC_A_TILE, ma, (kb0 + kk) * TC_KB_BYTES, (int)row, &sh->full[slot]);
            if (leader) bulk_g2s(st + FU_OFF_SFA + a * KS * TC_SF_TILE, sfa_src, KS * TC_SF_TILE, &sh->full[slot]);
        }
        if (DOWN && s == 0 && wait_unit) {
            // The unit's intermediate rows are complete when every gate_up tile of the unit has reported.  Normally the
            // caller has seen that already (one item ahead, off the critical path); otherwise wait here, with the
            // weight tiles above already on their way.
            const bool done = wait_counter(&p.ws.unit_done[it.unit], p.tiles_g * 4);
            if (!__all_sync(0xffffffffu, done)) return false;      // the stage never completes: consumers time out and unwind
        }
        if (!DOWN && wait_quant) {
            // the slot-ordered activation rows are written by this kernel's epilogue warps (all CTAs' together) while
            // the first weight tiles above are in flight
            const int nblk = p.has_ep_permute ? p.ep_permute.src_base[p.ep_permute.world] * (p.hidden / SF_BLOCK) : p.pq_blocks;
            const bool done = wait_counter(&p.ws.counters[CNT_PQ_DONE], (nblk + FU_PQ_CHUNK - 1) / FU_PQ_CHUNK);
            if (!__all_sync(0xffffffffu, done)) return false;
            wait_quant = false;
        }
        // tokens and their scale atoms
#pragma unroll
        for (int kk = 0; kk < KS; ++kk)
            if (leader) tma_load_2d(st + FU_OFF_B + kk * FU_B_TILE, mb, (kb0 + kk) * TC_KB_BYTES, u.y, &sh->full[slot]);
        if (leader) bulk_g2s(st + FU_OFF_SFB, sfb + ((size_t)it.unit * (K / 64) + (size_t)kb0 * 4) * 512, KS * TC_SF_TILE, &sh->full[slot]);
        ++g;
    }
    return true;
}

__device__ __forceinline__ void fu_producer(const FuParams& p, uint8_t* smem, FuShared* sh) {
    const bool leader = elect_one();
    const int leader_lane = __ffs(__ballot_sync(0xffffffffu, leader)) - 1;
    const bool do_g = p.phases & TC_PHASE_GATE_UP, do_d = p.phases & TC_PHASE_DOWN;
    // The first item of a CTA is its block index.  Its unit record is requested together with the unit count,
    // on the assumption that it belongs to the first kind of item in the queue (no dependent round trip in
    // front of the first copy); the queue hands out the items from gridDim.x on.
    const int tiles_first = do_g ? p.tiles_g : p.tiles_d;
    const int spec_unit = (int)blockIdx.x / tiles_first;
    int4 spec_u = make_int4(0, 0, 0, 8);
    if (spec_unit < p.ws.tc_unit_capacity) spec_u = p.ws.tc_units[spec_unit];
    const int num_units = min(p.ws.counters[CNT_TC_UNITS], p.ws.tc_unit_capacity);
    const long long total_g = do_g ? (long long)num_units * p.tiles_g : 0;
    const long long total = total_g + (do_d ? (long long)num_units * p.tiles_d : 0);
    if (leader && num_units >= 0) VMOE_MARK_MIN(p.ws, 11);
    auto decode = [&](long long item) -> FuItem {
        if (item < total_g) return FuItem{ITEM_GATE_UP, (int)(item / p.tiles_g), (int)(item % p.tiles_g)};
        const long long i2 = item - total_g;
        return FuItem{ITEM_DOWN, (int)(i2 / p.tiles_d), (int)(i2 % p.tiles_d)};
    };
    auto pop = [&]() -> long long {
        long long v = 0;
        if (leader) v = (long long)atomicAdd(&p.ws.counters[p.queue], 1) + gridDim.x;
        return __shfl_sync(0xffffffffu, v, leader_lane);
    };
    auto alpha_of = [&](const FuItem& it, const int4& u) -> float {
        const bool shd = u.x >= p.E;
        if (it.kind == ITEM_GATE_UP) return shd ? p.gs13_shared[0] : p.gs13_routed[u.x];
        return shd ? p.gs2_shared[0] : p.gs2_routed[u.x];
    };
    long long next = blockIdx.x;
    FuItem next_it = decode(next < total ? next : 0);
    int4 next_u = make_int4(0, 0, 0, 8);
    if (next < total) next_u = (next_it.unit == spec_unit) ? spec_u : p.ws.tc_units[next_it.unit];
    // the expert's global scale travels to the epilogue with the item's last stage record; like the unit record it
    // is requested one item ahead (after the current item's copies are out)
    float next_alpha = (next < total) ? alpha_of(next_it, next_u) : 0.f;
    const bool wait_units = do_g && do_d;
    // Is the next item's unit complete already?  Asked with an acquire load one item ahead, after the current item's
    // copies are out: in the steady state every down item finds its unit complete and never waits inside its stages.
    auto unit_ready = [&](const FuItem& it) -> bool {
        if (!wait_units || it.kind != ITEM_DOWN) return true;
        return ld_acquire_gpu(&p.ws.unit_done[it.unit]) >= p.tiles_g * 4;
    };
    bool next_ready = (next < total) ? unit_ready(next_it) : true;
    uint32_t g = 0;
    bool ok = true;
    bool wait_quant = p.pq_blocks > 0 || p.has_ep_permute;
    while (ok) {
        if (next >= total) break;
        const FuItem it = next_it;
        const int4 u = next_u;
        const float alpha = next_alpha;
        const bool ready = next_ready;
        // the pop and the unit record of the NEXT item are requested before this item's copies go out
        next = pop();
        next_it = decode(next < total ? next : 0);
        next_u = (next < total) ? p.ws.tc_units[next_it.unit] : make_int4(0, 0, 0, 8);
        if (it.kind == ITEM_GATE_UP) ok = fu_produce_item<2, 1>(p, smem, sh, leader, g, it, u, alpha, false, wait_quant);
        else if (p.ks_d == 2)        ok = fu_produce_item<1, 2>(p, smem, sh, leader, g, it, u, alpha, !ready, wait_quant);
        else                         ok = fu_produce_item<1, 1>(p, smem, sh, leader, g, it, u, alpha, !ready, wait_quant);
        if (next < total) { next_alpha = alpha_of(next_it, next_u); next_ready = unit_ready(next_it); }
    }
    if (!ok && leader) fu_timeout(p.ws, sh);
    // end marker
    const int slot = g % FU_STAGES;
    bool w = ok;
    if (w && g >= (uint32_t)FU_STAGES) w = mbar_wait(&sh->empty[slot], ((g / FU_STAGES) - 1) & 1);
    w = __all_sync(0xffffffffu, w);
    if (leader) {
        if (w) {
            sh->info[slot] = TcStageInfo{-1, 0, 0, 0, 0, 0, 0, 1, 0.f, {0, 0, 0}};
            mbar_arrive(&sh->full[slot]);
        } else {
            fu_timeout(p.ws, sh);
        }
    }
}

// ---------------------------------------------------------------------------------
// MMA issuer.  The whole warp walks the loop with identical values and only the tcgen05 instructions are
// predicated on one elected lane: operands then stay warp-uniform and each instruction issues in ~10-20
// cycles; issued from inside a single-lane branch they cost ~50 cycles each (measured), which made this
// warp, not HBM, the limit.  The instruction sequence of a stage is fixed at compile time per kind of item.
// ---------------------------------------------------------------------------------
template <int NA, int KS>
__device__ __forceinline__ void fu_issue_stage(bool leader, uint32_t st16, uint32_t sfcol, uint32_t dcol, uint32_t idesc, int kb) {
    constexpr int NT = NA * KS;
#pragma unroll
    for (int t = 0; t < NT; ++t)          // weight scales: tile t = a * KS + kk -> columns +0, +16
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint64_t d = make_desc(st16 + ((FU_OFF_SFA + (t * 4 + j) * 512) >> 4), DESC_SF_HI);
            if (leader) tc_cp_sf(sfcol + t * 16 + j * 4, d);
        }
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)             // token scales -> columns +32, +48
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint64_t d = make_desc(st16 + ((FU_OFF_SFB + (kk * 4 + j) * 512) >> 4), DESC_SF_HI);
            if (leader) tc_cp_sf(sfcol + 32 + kk * 16 + j * 4, d);
        }
#pragma unroll
    for (int kk = 0; kk < KS; ++kk)
#pragma unroll
        for (int a = 0; a < NA; ++a)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint64_t da = make_desc(st16 + (((a * KS + kk) * TC_A_TILE + j * 32) >> 4) + DESC_SW128_LBO, DESC_SW128_HI);
                const uint64_t db = make_desc(st16 + ((FU_OFF_B + kk * FU_B_TILE + j * 32) >> 4) + DESC_SW128_LBO, DESC_SW128_HI);
                const uint32_t acc = (kb > 0 || kk > 0 || j > 0) ? 1u : 0u;
                if (leader) tc_mma(dcol + a * FU_UT, da, db, idesc, sfcol + (a * KS + kk) * 16 + j * 4, sfcol + 32 + kk * 16 + j * 4, acc);
            }
}

__device__ __forceinline__ void fu_mma(uint8_t* smem, FuShared* sh, uint32_t tmem, const Workspace& ws) {
    const bool leader = elect_one();
    uint32_t g = 0, it = 0, idesc = 0;
    const uint32_t smem16 = smem_u32(smem) >> 4;
    bool ok = true;
    const TcStageInfo end_rec{-1, 0, 0, 0, 0, 0, 0, 1, 0.f, {0, 0, 0}};
    while (ok) {
        const int buf = it % FU_NBUF;
        bool first = true, end = false;
        while (true) {
            const int slot = g % FU_STAGES;
            if (!__all_sync(0xffffffffu, mbar_wait(&sh->full[slot], (g / FU_STAGES) & 1))) { ok = false; break; }
            tc_fence_after();
            const TcStageInfo inf = ld_info(&sh->info[slot]);
            if (leader && g == 0) VMOE_MARK_MIN(ws, 12);
            if (leader && inf.pad[0] == ITEM_DOWN && inf.expert >= 0) VMOE_MARK_MIN(ws, 13);
            if (leader && inf.pad[0] == ITEM_GATE_UP && inf.expert >= 0) VMOE_MARK_MAX(ws, 14);
            if (first) {
                // the accumulator buffer must have been drained by the epilogue FU_NBUF items ago
                bool w = true;
                if (it >= (uint32_t)FU_NBUF) w = mbar_wait(&sh->tmem_empty[buf], ((it / FU_NBUF) - 1) & 1);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                tc_fence_after();
                first = false;
            }
            if (inf.expert < 0) { end = true; break; }
            // descriptors: only the 14-bit start-address field (bytes >> 4) differs between tiles
            const uint32_t st16 = smem16 + slot * (FU_STAGE_BYTES >> 4);
            const uint32_t sfcol = tmem + TC_SF_COL0 + (g & 1) * FU_SF_COLS;
            const uint32_t dcol = tmem + buf * FU_ACC_STRIDE;
            if (inf.kb == 0) idesc = idesc_nvf4(inf.nbox);
            if (inf.pad[0] == ITEM_GATE_UP) fu_issue_stage<2, 1>(leader, st16, sfcol, dcol, idesc, inf.kb);
            else if (inf.pad[1] == 2)       fu_issue_stage<1, 2>(leader, st16, sfcol, dcol, idesc, inf.kb);
            else                            fu_issue_stage<1, 1>(leader, st16, sfcol, dcol, idesc, inf.kb);
            if (leader) tc_commit(&sh->empty[slot]);       // stage (and its scale columns) reusable when these finish
            ++g;
            if (inf.last) { if (leader) sh->epi[buf] = inf; break; }
        }
        if (!ok || end) break;
        if (leader) {
            tc_commit(&sh->tmem_full[buf]);        // fires when every MMA of the item has finished
            mbar_arrive(&sh->tmem_full[buf]);      // releases the epi[] record
        }
        ++it;
    }
    if (!ok && leader) fu_timeout(ws, sh);
    // End of work (or a failed wait): every epilogue set gets an end record in its next buffer.  The first of the
    // two buffers was claimed above when the end marker arrived; the second is waited for here.
    for (int n = 0; n < FU_EPI_SETS; ++n) {
        const uint32_t i2 = it + n;
        const int buf = i2 % FU_NBUF;
        if (ok && n > 0 && i2 >= (uint32_t)FU_NBUF) {
            const bool w = __all_sync(0xffffffffu, mbar_wait(&sh->tmem_empty[buf], ((i2 / FU_NBUF) - 1) & 1));
            if (!w && leader) fu_timeout(ws, sh);
        }
        if (leader) {
            sh->epi[buf] = end_rec;
            tc_commit(&sh->tmem_full[buf]);
            mbar_arrive(&sh->tmem_full[buf]);
        }
    }
}

// ---------------------------------------------------------------------------------
// epilogue: two sets of four warps take the items in turn; inside a set each warp owns one TMEM lane quadrant
// (32 rows of the item's 128)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void fu_epilogue(const FuParams& p, FuShared* sh, uint32_t tmem, int warp, int lane) {
    const int quad = warp & 3;                        // TMEM lanes [32*quad, 32*quad + 32)
    const int set = (warp - 2) >> 2;                  // which epilogue set
    const int wq = (warp - 2) & 3;                    // warp inside the set
    const int row = quad * 32 + lane;                 // row of the 128-row tile
    const bool combine = p.out != nullptr;
    if (p.pq_blocks > 0 || p.has_ep_permute) {
        // The permuting activation quantiser (expert parallelism: the permutation of the rows that arrived): chunks of
        // 256 blocks (one per epilogue thread), chunk c on CTA c mod gridDim.x; the producers meanwhile stream the
        // first weight tiles and only wait for the count of finished chunks before their first token-tile copy.
        const int et = (warp - 2) * 32 + lane;                // epilogue thread index, 0 .. 255
        const int bpr = p.hidden / SF_BLOCK;
        const int nblk = p.has_ep_permute ? p.ep_permute.src_base[p.ep_permute.world] * bpr : p.pq_blocks;
        const int chunks = (nblk + FU_PQ_CHUNK - 1) / FU_PQ_CHUNK;
        int done = 0;
        if (p.has_ep_permute) {
            constexpr int NB = 4;                             // chunks a thread handles per batch of table reads
            for (int c = blockIdx.x; c < chunks; c += NB * gridDim.x) {
                long long bs[NB];
#pragma unroll
                for (int n = 0; n < NB; ++n) {
                    const int cn = c + n * gridDim.x;
                    const long long b = (long long)cn * FU_PQ_CHUNK + et;
                    bs[n] = (cn < chunks && b < nblk) ? b : -1;
                    if (cn < chunks) ++done;
                }
                ep_permute_blocks<NB>(p.ep_permute, bs, p.hidden, p.tc_cap, p.ws);
            }
        } else {
            for (int c = blockIdx.x; c < chunks; c += gridDim.x, ++done) {
                const int b = c * FU_PQ_CHUNK + et;
                if (b < nblk)
                    permute_quantize_block<true>(b, p.quant.x, p.M, p.hidden, p.T, p.E, p.has_shared, p.tc_cap, p.quant.topk_ids,
                                                 p.quant.expert_map, p.ws, p.quant.pre_q, p.quant.pre_sf);
            }
        }
        if (done) {
            fence_proxy_async();          // the rows are read by bulk copies (async proxy)
            asm volatile("bar.sync 1, %0;" ::"r"(FU_PQ_CHUNK) : "memory");
            if (et == 0) red_release_add(&p.ws.counters[CNT_PQ_DONE], done);
        }
    }
    if (combine) {
        // tokens that receive no row at all (no local expert, no shared expert): zeros (+ residual)
        for (int m = blockIdx.x; m < p.M; m += gridDim.x)
            if (p.ws.token_expect[m] == 0)
                for (int c = (set * 4 + wq) * 32 + lane; c < p.hidden / 4; c += FU_EPI_SETS * 128)
                    combine_element<false>((long long)m * (p.hidden / 4) + c, p.ws.pair_out, p.ws.pair_slot, p.ws.expert_offsets, 0,
                                           p.hidden, p.T, p.E, p.has_shared, p.residual, p.out);
    }
    uint32_t epi_phase = 0;
    for (uint32_t it = set;; it += FU_EPI_SETS) {
        const int buf = it % FU_NBUF;
        if (!mbar_wait(&sh->tmem_full[buf], (it / FU_NBUF) & 1)) { if (lane == 0) fu_timeout(p.ws, sh); break; }
        tc_fence_after();
        const TcStageInfo inf = sh->epi[buf];
        if (inf.expert < 0) break;
        const float alpha = inf.alpha;
        const uint32_t tacc = tmem + ((uint32_t)(quad * 32) << 16) + buf * FU_ACC_STRIDE;
        if (inf.pad[0] == ITEM_GATE_UP) {
            const int n = inf.tile * TC_ROWS + row;       // intermediate index of this lane
            for (int c0 = 0; c0 < inf.nbox; c0 += 8) {
                uint32_t gr[8], ur[8];
                tc_ld8(tacc + c0, gr);
                tc_ld8(tacc + FU_UT + c0, ur);
                tc_ld_wait();
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int t = c0 + c;
                    if (t >= inf.ntok) break;                  // warp-uniform: columns past the unit's tokens hold nothing
                    const float gate = __uint_as_float(gr[c]) * alpha, up = __uint_as_float(ur[c]) * alpha;
                    const float sw = up * silu(gate);
                    float gm = fabsf(sw);
#pragma unroll
                    for (int o = 1; o < 16; o <<= 1) gm = fmaxf(gm, __shfl_xor_sync(0xffffffffu, gm, o));
                    const uint8_t sb = e4m3_encode(fmaxf(gm / 6.0f, 1e-30f));
                    float sc = e4m3_decode(sb);
                    if (sc < 1e-30f) sc = 1e-30f;
                    const uint32_t nib = e2m1_encode(ScaleDivider(sc)(sw));
                    const uint32_t nb = __shfl_down_sync(0xffffffffu, nib, 1);
                    const size_t srow = (size_t)(inf.slot0 + t);
                    if ((lane & 1) == 0) p.ws.inter_q[srow * (p.N / 2) + (n >> 1)] = (uint8_t)(nib | (nb << 4));
                    if ((lane & 15) == 0) {
                        p.ws.inter_sf[srow * (p.N / 16) + (n >> 4)] = sb;   // linear copy (stage checks)
                        // scale of block n/16 of token row t, in the atom layout of the down GEMM's B operand
                        p.ws.inter_sf_atoms[((size_t)inf.unit * (p.N / 64) + (n >> 6)) * 512 + (t & 31) * 16 + (t >> 5) * 4 + ((n >> 4) & 3)] = sb;
                    }
                }
            }
            tc_fence_before();
            // publish: other CTAs' bulk copies (async proxy) read these rows once all four warps of every tile of the unit
            // have reported.  Each lane orders its generic-proxy stores against the async proxy; a release by one lane
            // after the warp barrier then covers the whole warp's stores.
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sh->tmem_empty[buf]);
                red_release_add(&p.ws.unit_done[inf.unit], 1);
            }
        } else {
            const int j = inf.tile * TC_ROWS + row;       // hidden index of this lane
            for (int c0 = 0; c0 < inf.nbox; c0 += 8) {
                uint32_t yr[8];
                tc_ld8(tacc + c0, yr);
                tc_ld_wait();
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const int t = c0 + c;
                    if (t < inf.ntok) {
                        const int srow = inf.slot0 + t;
                        const float scale = p.ws.scatter_weights[srow] * alpha;
                        // expert parallelism: the row goes straight to its owner's combine slab (peer store)
                        float* orow = p.ws.row_dst ? p.ws.row_dst[srow] : p.ws.pair_out + (size_t)srow * p.hidden;
                        orow[j] = scale * __uint_as_float(yr[c]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
            if (combine) {
                // All four warps of the set have stored their 32 columns of every token row of the unit; then warp q
                // reports tokens q, q + 4, ... (one lane each, all at once): the last report of a token -- all its
                // rows, this column tile -- sums the token's rows for these 128 columns in the combine's fixed order.
                if (lane == 0) mbar_arrive(&sh->epi_bar[set]);
                if (!mbar_wait(&sh->epi_bar[set], epi_phase & 1)) { if (lane == 0) fu_timeout(p.ws, sh); break; }
                ++epi_phase;
                const int t = wq + 4 * lane;
                int tok = 0, last = 0;
                if (t < inf.ntok) {
                    tok = p.ws.gather_idx[inf.slot0 + t];
                    const int expect = p.ws.token_expect[tok];
                    last = atom_acq_rel_add(&p.ws.token_done[(size_t)tok * p.tiles_d + inf.tile], 1) + 1 == expect;
                }
                unsigned todo = __ballot_sync(0xffffffffu, last);
                if (todo) __threadfence();
                while (todo) {
                    const int src = __ffs(todo) - 1;
                    todo &= todo - 1;
                    const int tk = __shfl_sync(0xffffffffu, tok, src);
                    combine_element<true>((long long)tk * (p.hidden / 4) + inf.tile * (TC_ROWS / 4) + lane, p.ws.pair_out,
                                          p.ws.pair_slot, p.ws.expert_offsets, 0, p.hidden, p.T, p.E, p.has_shared, p.residual, p.out);
                }
            }
        }
    }
}

__global__ void __launch_bounds__(FU_THREADS, 1)
tc_fused_kernel(const __grid_constant__ FuParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    FuShared* sh = reinterpret_cast<FuShared*>(smem + (size_t)FU_STAGES * FU_STAGE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) VMOE_MARK_MIN(p.ws, 8);

    if (tid == 0) {
        for (int i = 0; i < FU_STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
        for (int i = 0; i < FU_NBUF; ++i) { mbar_init(&sh->tmem_full[i], 2); mbar_init(&sh->tmem_empty[i], 4); }
        for (int i = 0; i < FU_EPI_SETS; ++i) mbar_init(&sh->epi_bar[i], 4);
        sh->abort_flag = 0;
        sh->last_cta = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (warp == 0 && lane < 8) {
        // the descriptors of the first copies: fetched while the previous kernel is still running
        const CUtensorMap* maps[8] = {&p.map_w13_routed, &p.map_w13_shared, &p.map_w2_routed, &p.map_w2_shared,
                                      &p.map_act[0], &p.map_act[1], &p.map_inter[0], &p.map_inter[1]};
        asm volatile("prefetch.tensormap [%0];" ::"l"(maps[lane]) : "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    if (tid == 0) VMOE_MARK_MIN(p.ws, 9);
    pdl_begin();
    if (tid == 0) VMOE_MARK_MIN(p.ws, 10);

    if (warp == 0) fu_producer(p, smem, sh);
    else if (warp == 1) fu_mma(smem, sh, tmem, p.ws);
    else fu_epilogue(p, sh, tmem, warp, lane);

    tc_fence_before();
    __syncthreads();
    if (tid == 0) VMOE_MARK_MAX(p.ws, 15);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
    }
    if (tid == 32) VMOE_MARK_MAX(p.ws, 16);
    if (p.has_signal) {
        // expert parallelism: the last CTA to leave tells every rank that this rank's rows are in place;
        // the value carries the call number and, in its lowest bit, whether this rank hit an error
        // The ticket orders memory at GPU scope (release: this CTA's peer stores, seen through the barrier above;
        // acquire: the other CTAs'); the one system-scope release is the flag store of the last CTA, which is cumulative
        // over all of that.  (A system-scope fence in every CTA cost ~9 us at the end of every call.)
        if (tid == 0) sh->last_cta = (atom_acq_rel_add(p.signal.ticket, 1) == (int)gridDim.x - 1);
        __syncthreads();
        if (sh->last_cta && tid < p.signal.world) {
            const int32_t call = *p.signal.epoch + 1;
            const int32_t bad = (*(volatile int32_t*)&p.ws.counters[CNT_STATUS]) != 0;
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.signal.flag[tid]), "r"(call * 2 + bad) : "memory");
        }
        if (sh->last_cta && tid == 0) *p.signal.ticket = 0;
    }
}

// ---------------------------------------------------------------------------------
// bf16 -> NVFP4 quantiser that writes rows in sorted-slot order (every token row goes to the slot
// of each of its pairs and to its shared-expert slot) and block scales in the 128-row x 4-scale
// atom layout of the tensor-core B operand, relative to the first slot of the row's work unit.
// Same arithmetic as quantize_kernel (…tma_ext.cu:249-279).
// ---------------------------------------------------------------------------------
template <bool BATCHED>
__global__ void __launch_bounds__(256)
permute_quantize_kernel(const __nv_bfloat16* __restrict__ x, int M, int K, int T, int E, int has_shared, int tc_cap,
                        const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map, Workspace ws,
                        const uint8_t* __restrict__ pre_q, const uint8_t* __restrict__ pre_sf) {
    pdl_begin();
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (long long)M * (K / SF_BLOCK)) return;
    permute_quantize_block<BATCHED>(b, x, M, K, T, E, has_shared, tc_cap, topk_ids, expert_map, ws, pre_q, pre_sf);
}

// linear block scales [rows, K/16] -> atoms [rows/128][K/64][32][4][4]; NaN patterns become 0x00
// (they decode to zero: …tma_ext.cu:48-55).  Returns through *bad the number of signed bytes.
__global__ void __launch_bounds__(256)
prep_sf_kernel(const uint8_t* __restrict__ sf, long long rows, int K, uint8_t* __restrict__ atoms, int* bad) {
    const int spr = K / SF_BLOCK;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * spr) return;
    const long long row = i / spr; const int kb = (int)(i % spr);
    uint8_t v = sf[i];
    if ((v & 0x7F) == 0x7F) v = 0;
    else if (v & 0x80) { atomicAdd(bad, 1); }
    const int r = (int)(row % TC_ROWS);
    atoms[((row / TC_ROWS) * (K / 64) + (kb >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = v;
}

// ---------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;

int get_encoder() {
    if (g_encode) return VMOE_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return VMOE_ERR_CUDA;
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    return VMOE_OK;
}

// 2-D byte tensor [rows, row_bytes], box [box_rows, 128 bytes], 128-byte swizzle.  Encoded maps are kept in a
// hash table keyed by (device, base, shape): a map depends on nothing else, so an entry never goes stale, and a
// forward call re-uses its maps instead of paying a driver call per map per launch.  A model of many layers
// holds about ten maps per layer; the table is emptied only if it ever reaches 65536 entries.
struct MapKey {
    int dev; const void* base; uint64_t row_bytes, rows; uint32_t box_rows;
    bool operator==(const MapKey& o) const {
        return dev == o.dev && base == o.base && row_bytes == o.row_bytes && rows == o.rows && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.base) * 0x9E3779B97F4A7C15ull;
        h ^= (k.rows + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
        h ^= (k.row_bytes * 31 + k.box_rows * 131 + (uint64_t)k.dev * 65537 + (h << 6) + (h >> 2));
        return (size_t)h;
    }
};
static std::mutex g_map_mutex;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
    int dev = 0;
    cudaGetDevice(&dev);
    const MapKey key{dev, base, row_bytes, rows, box_rows};
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *map = it->second; return VMOE_OK; }
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {TC_KB_BYTES, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VMOE_ERR_CUDA;
    if (g_map_cache.size() >= 65536) g_map_cache.clear();
    g_map_cache.emplace(key, *map);
    return VMOE_OK;
}

// Scale atoms as a 2-D tensor: rows of one 512-byte atom (128 words), box = the four atoms of one 256-element k-step.
int make_sf_map(CUtensorMap* map, const void* base, uint64_t atoms) {
    int dev = 0;
    cudaGetDevice(&dev);
    const MapKey key{dev, base, 512, atoms, 0x80000004u};
    std::lock_guard<std::mutex> lock(g_map_mutex);
    auto it = g_map_cache.find(key);
    if (it != g_map_cache.end()) { *map = it->second; return VMOE_OK; }
    const cuuint64_t dims[2] = {128, atoms};
    const cuuint64_t strides[1] = {512};
    const cuuint32_t box[2] = {128, 4};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VMOE_ERR_CUDA;
    if (g_map_cache.size() >= 65536) g_map_cache.clear();
    g_map_cache.emplace(key, *map);
    return VMOE_OK;
}

int tc_sm_count() {
    static int n = 0;
    if (n == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); if (n <= 0) n = 148; }
    return n;
}

int launch_permute_quantize(const vmoe_shape& s, const __nv_bfloat16* x, const int32_t* ids, const int32_t* expert_map,
                            int M, const Workspace& ws, cudaStream_t st, const uint8_t* pre_q, const uint8_t* pre_sf) {
    const long long nblocks = (long long)M * (s.hidden / SF_BLOCK);
    if (nblocks == 0) return VMOE_OK;
    const unsigned blocks = (unsigned)((nblocks + 255) / 256);
    if (blocks <= 1024)
        launch_pdl(permute_quantize_kernel<true>, blocks, 256u, 0, st, x, M, s.hidden, s.topk, s.num_experts,
                                                              s.has_shared, tc_unit_cap(s, M), ids, expert_map, ws, pre_q, pre_sf);
    else
        launch_pdl(permute_quantize_kernel<false>, blocks, 256u, 0, st, x, M, s.hidden, s.topk, s.num_experts,
                                                               s.has_shared, tc_unit_cap(s, M), ids, expert_map, ws, pre_q, pre_sf);
    return cuda_status(cudaGetLastError());
}

int launch_prep_sf(const uint8_t* sf, long long rows, int K, uint8_t* atoms, int* bad, cudaStream_t st) {
    const long long n = rows * (K / SF_BLOCK);
    if (n == 0) return VMOE_OK;
    prep_sf_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(sf, rows, K, atoms, bad);
    return cuda_status(cudaGetLastError());
}

// Kernel parameters of the fused kernel: tensor maps (cached), scale-atom pointers, shape.
static int fill_fu_params(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
                          const Workspace& ws, long long b_rows, int phases, FuParams* out) {
    int rc = get_encoder();
    if (rc) return rc;
    FuParams& p = *out;
    memset(&p, 0, sizeof(p));
    const int K = s.hidden, N = s.inter;
    if ((rc = make_map(&p.map_w13_routed, routed.w13, K / 2, (uint64_t)s.num_experts * 2 * N, TC_ROWS))) return rc;
    if ((rc = make_map(&p.map_w2_routed, routed.w2, N / 2, (uint64_t)s.num_experts * K, TC_ROWS))) return rc;
    if (s.has_shared) {
        if ((rc = make_map(&p.map_w13_shared, shared.w13, K / 2, 2 * N, TC_ROWS))) return rc;
        if ((rc = make_map(&p.map_w2_shared, shared.w2, N / 2, K, TC_ROWS))) return rc;
    } else { p.map_w13_shared = p.map_w13_routed; p.map_w2_shared = p.map_w2_routed; }
    const long long S = b_rows >= 0 ? b_rows : (long long)s.max_tokens * s.topk + (s.has_shared ? s.max_tokens : 0);
    const uint64_t srows = (uint64_t)(S > 0 ? S : 1);
    const uint32_t boxes[2] = {8, 16};
    for (int i = 0; i < 2; ++i) {
        if ((rc = make_map(&p.map_act[i], ws.act_q_sorted, K / 2, srows, boxes[i]))) return rc;
        if ((rc = make_map(&p.map_inter[i], ws.inter_q, N / 2, srows, boxes[i]))) return rc;
    }
    p.sfa13_routed = prep.w13_sf_atoms; p.sfa13_shared = prep.shared_w13_sf_atoms;
    p.sfa2_routed = prep.w2_sf_atoms;   p.sfa2_shared = prep.shared_w2_sf_atoms;
    p.gs13_routed = routed.w13_gs; p.gs13_shared = shared.w13_gs;
    p.gs2_routed = routed.w2_gs;   p.gs2_shared = shared.w2_gs;
    p.ws = ws; p.hidden = K; p.N = N; p.E = s.num_experts;
    p.tiles_g = N / TC_ROWS; p.tiles_d = K / TC_ROWS;
    p.ks_d = ((N / 256) % 2 == 0) ? 2 : 1;      // two k-blocks per stage when the reduction length allows
    p.phases = phases;
    p.queue = (phases == TC_PHASE_DOWN) ? CNT_QUEUE2 : CNT_QUEUE1;     // the stage entry points run the phases one after the other
    p.T = s.topk; p.has_shared = s.has_shared;
    return VMOE_OK;
}

int launch_tc(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
              int M, const Workspace& ws, cudaStream_t st, int phases, __nv_bfloat16* out, const __nv_bfloat16* residual,
              bool* combined, int unit_cap, long long b_rows, const TcEpSignal* signal, const TcQuant* quant, bool* quantized,
              const TcEpPermute* ep_permute, bool* ep_done) {
    if (combined) *combined = false;
    if (quantized) *quantized = false;
    if (ep_done) *ep_done = false;
    if (M == 0 && !signal) return VMOE_OK;
    const int cap = unit_cap > 0 ? unit_cap : tc_unit_cap(s, M);
    if (cap == TC_UNIT_TOK_PREFILL) {
        // VMOE_PF_PAIR: bit 0 runs the gate_up projection on CTA pairs (cta_group::2, vmoe_tc_pair.cu), bit 1 the down
        // projection.
        int rc = VMOE_OK;
        const int pairs = tuning("VMOE_PF_PAIR", 0);
        if (phases & TC_PHASE_GATE_UP) {
            bool done = false;
            if (pairs & 1) rc = launch_pair_gate_up(s, routed, shared, prep, M, ws, st, b_rows, &done);
            if (!rc && !done) rc = launch_pf_gate_up(s, routed, shared, prep, M, ws, st, b_rows);
        }
        if (!rc && (phases & TC_PHASE_DOWN)) {
            bool done = false;
            if ((pairs & 2) && !ws.pair_rows_bf16) rc = launch_pair_down(s, routed, shared, prep, M, ws, st, b_rows, &done);
            if (!rc && !done) rc = launch_pf_down(s, routed, shared, prep, M, ws, st, b_rows);
        }
        return rc;
    }
    FuParams p;
    int rc = fill_fu_params(s, routed, shared, prep, ws, b_rows, phases, &p);
    if (rc) return rc;
    // Both projections in one launch?  (0: two launches of this kernel, one phase each -- for comparison runs.)
    if (phases == (TC_PHASE_GATE_UP | TC_PHASE_DOWN) && !signal && tuning("VMOE_FUSE_PHASES", 1) == 0) {
        int rc = launch_tc(s, routed, shared, prep, M, ws, st, TC_PHASE_GATE_UP, nullptr, nullptr, nullptr, cap, b_rows, nullptr);
        return rc ? rc : launch_tc(s, routed, shared, prep, M, ws, st, TC_PHASE_DOWN, nullptr, nullptr, nullptr, cap, b_rows, nullptr);
    }
    // The combine inside the kernel saves a launch but adds a counter round trip to every down item: it pays while
    // the step is latency-bound.
    const bool fuse_combine = out != nullptr && phases == (TC_PHASE_GATE_UP | TC_PHASE_DOWN) && ws.row_dst == nullptr &&
                              M <= ws.small_tokens && M <= tuning("VMOE_FUSE_COMBINE_TOKENS", 2);
    if (fuse_combine) { p.out = out; p.residual = residual; }
    p.M = M;
    if (quant && phases == (TC_PHASE_GATE_UP | TC_PHASE_DOWN)) {
        p.quant = *quant; p.pq_blocks = M * (s.hidden / SF_BLOCK); p.tc_cap = cap;
        if (quantized) *quantized = true;
    }
    if (combined) *combined = fuse_combine;
    if (signal) { p.has_signal = 1; p.signal = *signal; }
    if (ep_permute) { p.has_ep_permute = 1; p.ep_permute = *ep_permute; p.tc_cap = cap; }
    if (ep_done) *ep_done = signal != nullptr && ep_permute != nullptr;
    const size_t smem = (size_t)FU_STAGES * FU_STAGE_BYTES + sizeof(FuShared) + 1024;
    static bool attr_set[64] = {false};       // per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(tc_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return VMOE_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const long long units_hint = min((long long)M * s.topk + (s.has_shared ? M : 0), (long long)ws.tc_unit_capacity);
    const int per_unit = ((phases & TC_PHASE_GATE_UP) ? p.tiles_g : 0) + ((phases & TC_PHASE_DOWN) ? p.tiles_d : 0);
    long long grid = min((long long)tc_sm_count(), units_hint * per_unit);
    if (grid < 1) grid = 1;
    launch_pdl(tc_fused_kernel, (unsigned)grid, (unsigned)FU_THREADS, smem, st, p);
    return cuda_status(cudaGetLastError());
}

}  // namespace vmoe
