// Tensor-core path: block-scaled tcgen05.mma (kind::mxf4nvf4, 16-element E4M3 scales) grouped
// GEMM over the permutation tables, accumulators in TMEM.
//
//   tc_gemm_kernel<2> : gate_up projection (a8) + x alpha1 + SiLU*mul + FP4 re-quantisation (a9)
//   tc_gemm_kernel<1> : down projection (a10) + (router weight x alpha2) scaling per sorted slot
//
// Operand roles are swapped with respect to the usual token-major GEMM: the 128 rows of the
// UMMA tile are WEIGHT rows (A operand, streamed once from HBM by TMA with the 128-byte swizzle),
// the N dimension (8..64) holds the tokens routed to the expert (B operand, rows of the slot-
// ordered activation matrix).  With few tokens per expert this is a tensor-core GEMV: the FP4
// decode happens inside the tensor core instead of on the conversion (XU) pipe, which a CUDA-core
// GEMV saturates long before HBM does.  The same kernel serves prefill with more tokens per unit.
//
// Math follows fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:323-538 of the reference.
// Warp roles per persistent CTA: warp 0 = TMA / bulk-copy producer, warp 1 = MMA issuer and TMEM
// owner, warps 2-5 = epilogue (one TMEM lane quadrant each).  Every wait is bounded.
#include "vmoe_tc_common.cuh"
#include "vmoe_phases.cuh"

#include <string.h>

#include <mutex>
#include <vector>

#include <cuda.h>
#include <cudaTypedefs.h>

namespace vmoe {

// NA = weight matrices per item (2: gate + up, 1: down); KS = 128-byte k-blocks per stage; UT = tokens
// per unit (UMMA N <= UT).  A stage holds NA*KS weight tiles, KS token tiles and their scale atoms.
template <int NA, int KS, int UT> struct TcCfg {
    static constexpr int NT = NA * KS;
    static constexpr int B_TILE = UT * TC_KB_BYTES;
    static constexpr int STAGE_BYTES = NT * (TC_A_TILE + TC_SF_TILE) + KS * (B_TILE + TC_SF_TILE);
    static constexpr int STAGES = (TC_SMEM_BUDGET / STAGE_BYTES) > 12 ? 12 : (TC_SMEM_BUDGET / STAGE_BYTES);
    static constexpr int OFF_B = NT * TC_A_TILE;                 // [KS][UT x 128]
    static constexpr int OFF_SFA = OFF_B + KS * B_TILE;           // [NA][KS][4 atoms]
    static constexpr int OFF_SFB = OFF_SFA + NT * TC_SF_TILE;     // [KS][4 atoms]
    static constexpr int SF_COLS = (NT + KS) * 16;                // TMEM columns of one stage's scales
    // accumulator buffers in TMEM: short items (down) run further ahead of their epilogue
    static constexpr int ACC_STRIDE = NA * UT;
    static constexpr int NBUF = (256 / ACC_STRIDE) > 4 ? 4 : (256 / ACC_STRIDE);
    static_assert(TC_SF_COL0 + 2 * SF_COLS <= TC_TMEM_COLS, "scale columns do not fit");
};

struct TcParams {
    CUtensorMap map_a_routed, map_a_shared;    // weights [rows, K/2] bytes, box 128 x 128, swizzle 128B
    CUtensorMap map_b[4];                      // activations [slots, K/2] bytes, box 128 x {8,16,32,64}
    const uint8_t* sfa_routed; const uint8_t* sfa_shared;   // scale atoms [rows/128][K/64][512]
    const uint8_t* sfb;                         // per-unit scale atoms [unit][K/64][512]
    const float* gs_routed; const float* gs_shared;
    Workspace ws;
    int K;            // reduction length in elements
    int rows;         // weight rows per expert matrix (2N for gate_up, hidden for down)
    int N;            // intermediate size
    int hidden;
    int E;
    int tiles;        // items per unit
    int queue;        // counter index of the work queue
    int unit_capacity;   // entries of ws.tc_units
};

// ---------------------------------------------------------------------------------
// The kernel.  NA = 2: gate_up (A0 = gate rows, A1 = up rows of the same 128-n tile);
//              NA = 1: down.
// ---------------------------------------------------------------------------------
// Cycle counters per role, summed over CTAs (development aid, same slots as the large-batch kernels):
// [0] MMA: waiting for a full stage, [1] MMA: waiting for an accumulator buffer, [2] MMA: issuing,
// [3] epilogue warp 2: waiting, [4] epilogue warp 2: working, [5] producer: waiting for a slot, [6] items, [7] stages.
__device__ unsigned long long g_tc_prof[8];

// The three warp roles of one GEMM phase over an initialised ring (mbarriers at phase 0, TMEM allocated).
// Returns when every role has finished its last item; the caller synchronises the CTA afterwards.
template <int NA, int KS, int UT>
__device__ __forceinline__ void tc_roles(const TcParams& p, uint8_t* smem, TcShared* sh, uint32_t tmem, int warp, int lane) {
    using Cfg = TcCfg<NA, KS, UT>;
    if (warp == 0) {
        // ------------------------------------------------------------- producer (warp-uniform, see the MMA issuer)
        const bool leader = elect_one();
        const int leader_lane = __ffs(__ballot_sync(0xffffffffu, leader)) - 1;
        const int num_units = p.ws.counters[CNT_TC_UNITS];
        const long long total = (long long)num_units * p.tiles;
        const int kblocks = p.K / 256;
        uint32_t g = 0;
        bool ok = true;
        long long prof_wait = 0;
        // The first item of a CTA is its block index, so its unit record is requested together with the
        // unit count (no queue pop, no dependent round trip in front of the first copy); the queue hands
        // out the items from gridDim.x on.  The pop and the unit record of the NEXT item are requested
        // before the loads of the current one are issued.
        auto pop = [&]() -> long long {
            long long v = 0;
            if (leader) v = (long long)atomicAdd(&p.ws.counters[p.queue], 1) + gridDim.x;
            return __shfl_sync(0xffffffffu, v, leader_lane);
        };
        long long next = blockIdx.x;
        int4 next_u = make_int4(0, 0, 0, 8);
        if (next / p.tiles < p.unit_capacity) next_u = p.ws.tc_units[next / p.tiles];    // independent of the unit count
        if (next >= total) next_u = make_int4(0, 0, 0, 8);
        // the expert's global scale travels to the epilogue with the item's last stage record; like the unit
        // record it is requested one item ahead (after the current item's copies are out)
        float next_alpha = (next_u.x >= p.E) ? p.gs_shared[0] : p.gs_routed[next_u.x];
        while (ok) {
            const long long item = next;
            if (item >= total) break;
            // unit-major order: consecutive items are the row tiles of one unit
            const int unit = (int)(item / p.tiles), tile = (int)(item % p.tiles);
            const int4 u = next_u;
            const float alpha = next_alpha;
            next = pop();
            next_u = (next < total) ? p.ws.tc_units[next / p.tiles] : make_int4(0, 0, 0, 8);
            const bool shd = u.x >= p.E;
            const int e = shd ? 0 : u.x;
            const CUtensorMap* ma = shd ? &p.map_a_shared : &p.map_a_routed;
            const uint8_t* sfa = shd ? p.sfa_shared : p.sfa_routed;
            const int nbox = u.w;
            const CUtensorMap* mb = &p.map_b[nbox == 8 ? 0 : nbox == 16 ? 1 : nbox == 32 ? 2 : 3];
            const int steps = kblocks / KS;
            for (int ks = 0; ks < steps; ++ks) {
                const int slot = g % Cfg::STAGES;
                const long long tw0 = prof_clock();
                bool w = true;
                if (g >= (uint32_t)Cfg::STAGES) w = mbar_wait(&sh->empty[slot], ((g / Cfg::STAGES) - 1) & 1);
                w = w && !(*(volatile int*)&sh->abort_flag);
                if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                prof_wait += prof_clock() - tw0;
                uint8_t* st = smem + (size_t)slot * Cfg::STAGE_BYTES;
                const uint32_t bytes = Cfg::NT * (TC_A_TILE + TC_SF_TILE) + KS * (nbox * TC_KB_BYTES + TC_SF_TILE);
                const int kb0 = ks * KS;                       // first k-block of this stage
                if (leader) {
                    sh->info[slot] = TcStageInfo{u.x, u.y, u.z, nbox, tile, unit, ks, ks == steps - 1, ks == steps - 1 ? alpha : 0.f, {0, 0, 0}};
                    mbar_arrive_expect_tx(&sh->full[slot], bytes);
                }
#pragma unroll
                for (int a = 0; a < NA; ++a) {
                    // gate_up: A0 = rows [tile*128, +128) of the gate half, A1 = same rows of the up half
                    const int row_in_expert = (NA == 2 ? a * p.N : 0) + tile * TC_ROWS;
                    const long long row = (long long)e * p.rows + row_in_expert;
                    // the atoms of consecutive k-blocks of one row tile are contiguous
                    const uint8_t* sfa_src = sfa + ((size_t)(row / TC_ROWS) * (p.K / 64) + (size_t)kb0 * 4) * 512;
#pragma unroll
                    for (int kk = 0; kk < KS; ++kk)
                        if (leader) tma_load_2d(st + (a * KS + kk) * TC_A_TILE, ma, (kb0 + kk) * TC_KB_BYTES, (int)row, &sh->full[slot]);
                    if (leader) bulk_g2s(st + Cfg::OFF_SFA + a * KS * TC_SF_TILE, sfa_src, KS * TC_SF_TILE, &sh->full[slot]);
                }
                const uint8_t* sfb_src = p.sfb + ((size_t)unit * (p.K / 64) + (size_t)kb0 * 4) * 512;
#pragma unroll
                for (int kk = 0; kk < KS; ++kk)
                    if (leader) tma_load_2d(st + Cfg::OFF_B + kk * Cfg::B_TILE, mb, (kb0 + kk) * TC_KB_BYTES, u.y, &sh->full[slot]);
                if (leader) bulk_g2s(st + Cfg::OFF_SFB, sfb_src, KS * TC_SF_TILE, &sh->full[slot]);
                ++g;
            }
            next_alpha = (next_u.x >= p.E) ? p.gs_shared[0] : p.gs_routed[next_u.x];
        }
        if (leader) {
            if (!ok) tc_timeout(p.ws, sh);
            VMOE_PROF_ADD(&g_tc_prof[5], prof_wait);
            VMOE_PROF_ADD(&g_tc_prof[7], g);
        }
        // end marker
        const int slot = g % Cfg::STAGES;
        bool w = true;
        if (g >= (uint32_t)Cfg::STAGES) w = mbar_wait(&sh->empty[slot], ((g / Cfg::STAGES) - 1) & 1);
        w = __all_sync(0xffffffffu, w);
        if (leader) {
            if (w) {
                sh->info[slot] = TcStageInfo{-1, 0, 0, 0, 0, 0, 0, 1};
                mbar_arrive(&sh->full[slot]);
            } else {
                tc_timeout(p.ws, sh);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer
        // The whole warp walks the loop with identical values and only the tcgen05 instructions are
        // predicated on one elected lane: operands then stay warp-uniform and each instruction issues
        // in ~10-20 cycles; issued from inside a single-lane branch they cost ~50 cycles each
        // (measured), which made this warp, not HBM, the limit.
        const bool leader = elect_one();
        uint32_t g = 0, it = 0, idesc = 0;
        const uint32_t smem16 = smem_u32(smem) >> 4;
        bool ok = true;
        long long pw_full = 0, pw_acc = 0, p_issue = 0;
        while (ok) {
            const int buf = it % Cfg::NBUF;
            bool first = true;
            bool end = false;
            while (true) {
                const int slot = g % Cfg::STAGES;
                const long long c0 = prof_clock();
                if (!__all_sync(0xffffffffu, mbar_wait(&sh->full[slot], (g / Cfg::STAGES) & 1))) { ok = false; break; }
                const long long c1 = prof_clock();
                pw_full += c1 - c0;
                tc_fence_after();
                const TcStageInfo inf = ld_info(&sh->info[slot]);
                if (first) {
                    // the accumulator buffer must have been drained by the epilogue NBUF items ago
                    bool w = true;
                    if (it >= (uint32_t)Cfg::NBUF) w = mbar_wait(&sh->tmem_empty[buf], ((it / Cfg::NBUF) - 1) & 1);
                    if (!__all_sync(0xffffffffu, w)) { ok = false; break; }
                    pw_acc += prof_clock() - c1;
                    tc_fence_after();
                    first = false;
                }
                if (inf.expert < 0) {
                    if (leader) sh->epi[buf] = inf;
                    end = true;
                    break;
                }
                const long long c2 = prof_clock();
                // descriptors: only the 14-bit start-address field (bytes >> 4) differs between
                // tiles, so each one is a single add on a per-stage base
                const uint32_t st16 = smem16 + slot * (Cfg::STAGE_BYTES >> 4);
                const uint32_t sfcol = tmem + TC_SF_COL0 + (g & 1) * Cfg::SF_COLS;
#pragma unroll
                for (int t = 0; t < Cfg::NT; ++t)          // weight scales: tile t = a * KS + kk
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t d = make_desc(st16 + ((Cfg::OFF_SFA + (t * 4 + j) * 512) >> 4), DESC_SF_HI);
                        if (leader) tc_cp_sf(sfcol + t * 16 + j * 4, d);
                    }
#pragma unroll
                for (int kk = 0; kk < KS; ++kk)             // token scales
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint64_t d = make_desc(st16 + ((Cfg::OFF_SFB + (kk * 4 + j) * 512) >> 4), DESC_SF_HI);
                        if (leader) tc_cp_sf(sfcol + Cfg::NT * 16 + kk * 16 + j * 4, d);
                    }
                if (inf.kb == 0) idesc = idesc_nvf4(inf.nbox);
                const uint32_t dcol = tmem + buf * Cfg::ACC_STRIDE;
#pragma unroll
                for (int kk = 0; kk < KS; ++kk)
#pragma unroll
                    for (int a = 0; a < NA; ++a)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const uint64_t da = make_desc(st16 + (((a * KS + kk) * TC_A_TILE + j * 32) >> 4) + DESC_SW128_LBO, DESC_SW128_HI);
                            const uint64_t db = make_desc(st16 + ((Cfg::OFF_B + kk * Cfg::B_TILE + j * 32) >> 4) + DESC_SW128_LBO, DESC_SW128_HI);
                            const uint32_t acc = (inf.kb > 0 || kk > 0 || j > 0) ? 1u : 0u;
                            if (leader) tc_mma(dcol + a * UT, da, db, idesc, sfcol + (a * KS + kk) * 16 + j * 4,
                                               sfcol + Cfg::NT * 16 + kk * 16 + j * 4, acc);
                        }
                if (leader) tc_commit(&sh->empty[slot]);       // stage (and its scale columns) reusable when these finish
                p_issue += prof_clock() - c2;
                ++g;
                if (inf.last) { if (leader) sh->epi[buf] = inf; break; }
            }
            if (!ok) break;
            if (leader) {
                tc_commit(&sh->tmem_full[buf]);        // fires when every MMA of the item has finished
                mbar_arrive(&sh->tmem_full[buf]);      // releases the epi[] record
            }
            ++it;
            if (end) break;
        }
        if (leader) {
            VMOE_PROF_ADD(&g_tc_prof[0], pw_full);
            VMOE_PROF_ADD(&g_tc_prof[1], pw_acc);
            VMOE_PROF_ADD(&g_tc_prof[2], p_issue);
            VMOE_PROF_ADD(&g_tc_prof[6], it);
        }
        if (!ok && leader) {
            tc_timeout(p.ws, sh);
            // let the epilogue leave
            sh->epi[it % Cfg::NBUF] = TcStageInfo{-1, 0, 0, 0, 0, 0, 0, 1};
            tc_commit(&sh->tmem_full[it % Cfg::NBUF]);
            mbar_arrive(&sh->tmem_full[it % Cfg::NBUF]);
        }
    } else {
        // ------------------------------------------------------------- epilogue
        const int quad = warp & 3;                        // TMEM lanes [32*quad, 32*quad + 32)
        const int row = quad * 32 + lane;                 // row of the 128-row tile
        uint32_t it = 0;
        long long pe_wait = 0, pe_work = 0;
        while (true) {
            const int buf = it % Cfg::NBUF;
            const long long c0 = prof_clock();
            if (!mbar_wait(&sh->tmem_full[buf], (it / Cfg::NBUF) & 1)) { if (lane == 0) tc_timeout(p.ws, sh); break; }
            const long long c1 = prof_clock();
            pe_wait += c1 - c0;
            tc_fence_after();
            const TcStageInfo inf = sh->epi[buf];
            if (inf.expert < 0) break;
            const float alpha = inf.alpha;
            const uint32_t tacc = tmem + ((uint32_t)(quad * 32) << 16) + buf * Cfg::ACC_STRIDE;
            if (NA == 2) {
                const int n = inf.tile * TC_ROWS + row;       // intermediate index of this lane
                for (int c0 = 0; c0 < inf.nbox; c0 += 8) {
                    uint32_t gr[8], ur[8];
                    tc_ld8(tacc + c0, gr);
                    tc_ld8(tacc + UT + c0, ur);
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
                        {
                            const size_t srow = (size_t)(inf.slot0 + t);
                            if ((lane & 1) == 0) p.ws.inter_q[srow * (p.N / 2) + (n >> 1)] = (uint8_t)(nib | (nb << 4));
                            if ((lane & 15) == 0) p.ws.inter_sf[srow * (p.N / 16) + (n >> 4)] = sb;   // linear copy (stage checks)
                            if ((lane & 15) == 0)   // scale of block n/16 of token row t, in the atom layout of the down GEMM's B operand
                                p.ws.inter_sf_atoms[((size_t)inf.unit * (p.N / 64) + (n >> 6)) * 512 + (t & 31) * 16 + (t >> 5) * 4 + ((n >> 4) & 3)] = sb;
                        }
                    }
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
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->tmem_empty[buf]);
            pe_work += prof_clock() - c1;
            ++it;
        }
        if (warp == 2 && lane == 0) {
            VMOE_PROF_ADD(&g_tc_prof[3], pe_wait);
            VMOE_PROF_ADD(&g_tc_prof[4], pe_work);
        }
    }
}

template <int NA, int KS, int UT>
__device__ __forceinline__ void tc_init_barriers(TcShared* sh) {
    using Cfg = TcCfg<NA, KS, UT>;
    for (int i = 0; i < Cfg::STAGES; ++i) { mbar_init(&sh->full[i], 1); mbar_init(&sh->empty[i], 1); }
    for (int i = 0; i < Cfg::NBUF; ++i) { mbar_init(&sh->tmem_full[i], 2); mbar_init(&sh->tmem_empty[i], 4); }
    sh->abort_flag = 0;
    mbar_fence_init();
}

template <int NA, int KS, int UT>
__global__ void __launch_bounds__(TC_THREADS, 1)
tc_gemm_kernel(const __grid_constant__ TcParams p) {
    using Cfg = TcCfg<NA, KS, UT>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    TcShared* sh = reinterpret_cast<TcShared*>(smem + (size_t)Cfg::STAGES * Cfg::STAGE_BYTES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) tc_init_barriers<NA, KS, UT>(sh);
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    pdl_begin();

    tc_roles<NA, KS, UT>(p, smem, sh, tmem, warp, lane);

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TC_TMEM_COLS) : "memory");
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
                        const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map, Workspace ws) {
    pdl_begin();
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= (long long)M * (K / SF_BLOCK)) return;
    permute_quantize_block<BATCHED>(b, x, M, K, T, E, has_shared, tc_cap, topk_ids, expert_map, ws);
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

// 2-D byte tensor [rows, row_bytes], box [box_rows, 128 bytes], 128-byte swizzle.  Encoded maps are
// kept in a small cache keyed by (device, base, shape): a forward call re-uses them instead of
// paying a driver call per map per launch.
struct MapKey { int dev; const void* base; uint64_t row_bytes, rows; uint32_t box_rows; };
struct MapEntry { MapKey key; CUtensorMap map; };
static std::mutex g_map_mutex;
static std::vector<MapEntry> g_map_cache;

int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_map_mutex);
    for (const MapEntry& e : g_map_cache)
        if (e.key.dev == dev && e.key.base == base && e.key.row_bytes == row_bytes && e.key.rows == rows && e.key.box_rows == box_rows) {
            *map = e.map;
            return VMOE_OK;
        }
    const cuuint64_t dims[2] = {row_bytes, rows};
    const cuuint64_t strides[1] = {row_bytes};
    const cuuint32_t box[2] = {TC_KB_BYTES, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return VMOE_ERR_CUDA;
    if (g_map_cache.size() >= 256) g_map_cache.erase(g_map_cache.begin());
    g_map_cache.push_back(MapEntry{MapKey{dev, base, row_bytes, rows, box_rows}, *map});
    return VMOE_OK;
}

int tc_sm_count() {
    static int n = 0;
    if (n == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); if (n <= 0) n = 148; }
    return n;
}

int launch_permute_quantize(const vmoe_shape& s, const __nv_bfloat16* x, const int32_t* ids, const int32_t* expert_map,
                            int M, const Workspace& ws, cudaStream_t st) {
    const long long nblocks = (long long)M * (s.hidden / SF_BLOCK);
    if (nblocks == 0) return VMOE_OK;
    const unsigned blocks = (unsigned)((nblocks + 255) / 256);
    if (blocks <= 1024)
        launch_pdl(permute_quantize_kernel<true>, blocks, 256u, 0, st, x, M, s.hidden, s.topk, s.num_experts,
                                                              s.has_shared, tc_unit_cap(s, M), ids, expert_map, ws);
    else
        launch_pdl(permute_quantize_kernel<false>, blocks, 256u, 0, st, x, M, s.hidden, s.topk, s.num_experts,
                                                               s.has_shared, tc_unit_cap(s, M), ids, expert_map, ws);
    return cuda_status(cudaGetLastError());
}

int launch_prep_sf(const uint8_t* sf, long long rows, int K, uint8_t* atoms, int* bad, cudaStream_t st) {
    const long long n = rows * (K / SF_BLOCK);
    if (n == 0) return VMOE_OK;
    prep_sf_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(sf, rows, K, atoms, bad);
    return cuda_status(cudaGetLastError());
}

// Kernel parameters of one GEMM phase: tensor maps (cached), scale-atom pointers, shape.  UT = tokens per unit.
template <int NA>
static int fill_tc_params(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
                          const Workspace& ws, long long b_rows, int UT, TcParams* out) {
    int rc = get_encoder();
    if (rc) return rc;
    TcParams& p = *out;
    memset(&p, 0, sizeof(p));
    const int K = (NA == 2) ? s.hidden : s.inter;              // reduction length
    const int rows = (NA == 2) ? 2 * s.inter : s.hidden;       // weight rows per expert
    const uint8_t* wr = (NA == 2) ? routed.w13 : routed.w2;
    const uint8_t* wsx = (NA == 2) ? shared.w13 : shared.w2;
    if ((rc = make_map(&p.map_a_routed, wr, K / 2, (uint64_t)s.num_experts * rows, TC_ROWS))) return rc;
    if (s.has_shared) { if ((rc = make_map(&p.map_a_shared, wsx, K / 2, rows, TC_ROWS))) return rc; }
    else p.map_a_shared = p.map_a_routed;
    const long long S = b_rows >= 0 ? b_rows : (long long)s.max_tokens * s.topk + (s.has_shared ? s.max_tokens : 0);
    const uint8_t* bsrc = (NA == 2) ? ws.act_q_sorted : ws.inter_q;
    const int boxes[4] = {8, 16, 32, 64};
    for (int i = 0; i < 4 && boxes[i] <= UT; ++i)
        if ((rc = make_map(&p.map_b[i], bsrc, K / 2, (uint64_t)(S > 0 ? S : 1), boxes[i]))) return rc;
    p.sfa_routed = (NA == 2) ? prep.w13_sf_atoms : prep.w2_sf_atoms;
    p.sfa_shared = (NA == 2) ? prep.shared_w13_sf_atoms : prep.shared_w2_sf_atoms;
    p.sfb = (NA == 2) ? ws.act_sf_atoms : ws.inter_sf_atoms;
    p.gs_routed = (NA == 2) ? routed.w13_gs : routed.w2_gs;
    p.gs_shared = (NA == 2) ? shared.w13_gs : shared.w2_gs;
    p.ws = ws; p.K = K; p.rows = rows; p.N = s.inter; p.hidden = s.hidden; p.E = s.num_experts;
    p.tiles = (NA == 2) ? s.inter / TC_ROWS : s.hidden / TC_ROWS;
    p.queue = (NA == 2) ? CNT_QUEUE1 : CNT_QUEUE2;
    p.unit_capacity = max_tc_units(&s);
    return VMOE_OK;
}

template <int NA, int KS, int UT>
static int launch_tc(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
                     int M, const Workspace& ws, cudaStream_t st, long long b_rows) {
    using Cfg = TcCfg<NA, KS, UT>;
    TcParams p;
    int rc = fill_tc_params<NA>(s, routed, shared, prep, ws, b_rows, UT, &p);
    if (rc) return rc;
    const size_t smem = (size_t)Cfg::STAGES * Cfg::STAGE_BYTES + sizeof(TcShared) + 1024;
    static bool attr_set[64] = {false};       // per device, per instantiation
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        if (cudaFuncSetAttribute(tc_gemm_kernel<NA, KS, UT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return VMOE_ERR_CUDA;
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    const long long units_hint = min((long long)M * s.topk + (s.has_shared ? M : 0), (long long)max_tc_units(&s));
    long long grid = min((long long)tc_sm_count(), units_hint * p.tiles);
    if (grid < 1) grid = 1;
    launch_pdl(tc_gemm_kernel<NA, KS, UT>, (unsigned)grid, (unsigned)TC_THREADS, smem, st, p);
    return cuda_status(cudaGetLastError());
}

int launch_tc_gate_up(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
                      int M, const Workspace& ws, cudaStream_t st, int unit_cap, long long b_rows) {
    if (M == 0) return VMOE_OK;
    const int cap = unit_cap > 0 ? unit_cap : tc_unit_cap(s, M);
    if (cap == TC_UNIT_TOK_PREFILL) return launch_pf_gate_up(s, routed, shared, prep, M, ws, st, b_rows);
    const bool small = cap == TC_UNIT_TOK_SMALL;
    return small ? launch_tc<2, 1, TC_UNIT_TOK_SMALL>(s, routed, shared, prep, M, ws, st, b_rows)
                 : launch_tc<2, 1, TC_UNIT_TOK>(s, routed, shared, prep, M, ws, st, b_rows);
}
int launch_tc_down(const vmoe_shape& s, const WeightSet& routed, const WeightSet& shared, const PreparedSet& prep,
                   int M, const Workspace& ws, cudaStream_t st, int unit_cap, long long b_rows) {
    if (M == 0) return VMOE_OK;
    const int cap = unit_cap > 0 ? unit_cap : tc_unit_cap(s, M);
    if (cap == TC_UNIT_TOK_PREFILL) return launch_pf_down(s, routed, shared, prep, M, ws, st, b_rows);
    // two k-blocks per stage when the reduction length allows: half as many ring round trips per byte
    const bool small = cap == TC_UNIT_TOK_SMALL;
    if ((s.inter / 256) % 2 == 0)
        return small ? launch_tc<1, 2, TC_UNIT_TOK_SMALL>(s, routed, shared, prep, M, ws, st, b_rows)
                     : launch_tc<1, 2, TC_UNIT_TOK>(s, routed, shared, prep, M, ws, st, b_rows);
    return small ? launch_tc<1, 1, TC_UNIT_TOK_SMALL>(s, routed, shared, prep, M, ws, st, b_rows)
                 : launch_tc<1, 1, TC_UNIT_TOK>(s, routed, shared, prep, M, ws, st, b_rows);
}

int debug_read_tc_profile(unsigned long long* out8) {
    if (cudaMemcpyFromSymbol(out8, g_tc_prof, sizeof(g_tc_prof)) != cudaSuccess) return VMOE_ERR_CUDA;
    unsigned long long zero[8] = {0};
    return cuda_status(cudaMemcpyToSymbol(g_tc_prof, zero, sizeof(zero)));
}

}  // namespace vmoe
