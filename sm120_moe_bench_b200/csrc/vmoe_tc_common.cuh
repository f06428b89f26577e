// Pieces shared by the tensor-core kernels: constants, PTX wrappers (TMA, tcgen05, descriptors),
// the control block in shared memory and the host-side tensor-map helper.
#pragma once

#include "vmoe_common.cuh"

#include <cuda.h>

namespace vmoe {

constexpr int TC_THREADS = 192;
constexpr int TC_ROWS = 128;                 // weight rows per tile (UMMA M)
constexpr int TC_KB_BYTES = 128;             // bytes of K per row per stage = 256 E2M1 elements
constexpr int TC_A_TILE = TC_ROWS * TC_KB_BYTES;            // 16 KiB
constexpr int TC_SF_TILE = 4 * 512;                         // four 128-row x 4-scale atoms
constexpr int TC_TMEM_COLS = 512;
constexpr int TC_SF_COL0 = 256;              // first TMEM column of the scale-factor area

constexpr int TC_SMEM_BUDGET = 227 * 1024 - 3 * 1024;     // dynamic shared memory minus control block and alignment slack

struct alignas(16) TcStageInfo {   // kb = step index within the item; alpha = the expert's global scale (valid on the last step)
    int expert, slot0, ntok, nbox, tile, unit, kb, last;
    float alpha; int pad[3];
};

// Role cycle counters are a development aid: compiled in only with -DVMOE_PROFILE (the debug read-out then
// returns them; otherwise it returns zeros and the clock reads vanish from the kernels).
#ifdef VMOE_PROFILE
__device__ __forceinline__ long long prof_clock() { return clock64(); }
#define VMOE_PROF_ADD(ptr, v) atomicAdd((ptr), (unsigned long long)(v))
#else
__device__ __forceinline__ long long prof_clock() { return 0; }
#define VMOE_PROF_ADD(ptr, v) ((void)0)
#endif

struct TcShared {
    uint64_t full[12], empty[12];
    uint64_t tmem_full[4], tmem_empty[4];
    TcStageInfo info[12];
    TcStageInfo epi[4];
    uint32_t tmem_base;
    int abort_flag;
};


// ---------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------
// Stage record written by the producer lane and read by every lane of the MMA warp after the stage's
// mbarrier completed: three 16-byte volatile loads.
__device__ __forceinline__ TcStageInfo ld_info(const TcStageInfo* src) {
    TcStageInfo r;
    const uint32_t a = smem_u32(src);
    asm volatile("ld.volatile.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.expert), "=r"(r.slot0), "=r"(r.ntok), "=r"(r.nbox) : "r"(a) : "memory");
    asm volatile("ld.volatile.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.tile), "=r"(r.unit), "=r"(r.kb), "=r"(r.last) : "r"(a + 16) : "memory");
    asm volatile("ld.volatile.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.alpha), "=r"(r.pad[0]), "=r"(r.pad[1]), "=r"(r.pad[2]) : "r"(a + 32) : "memory");
    return r;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)) : "memory");
}
// One lane of a fully converged warp, chosen by the hardware (elect.sync): the predicate under which
// single-thread asynchronous instructions (TMA, tcgen05.cp / mma / commit) are issued.
__device__ __forceinline__ bool elect_one() {
    uint32_t leader;
    asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(leader));
    return leader != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
        ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptors (sm_100 format: version 1 in bits 46-47)
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    // K-major, 128-byte swizzle: rows are 128 bytes apart, 8-row groups 1024 bytes apart
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
    // no swizzle: 32 rows of 16 bytes, 8-row groups 128 bytes apart
    return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
// the same descriptors as (low word = start address >> 4 | LBO << 16, constant high word)
constexpr uint32_t DESC_SW128_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
constexpr uint32_t DESC_SF_HI = (128u >> 4) | (1u << 14);
constexpr uint32_t DESC_SW128_LBO = 1u << 16;
__device__ __forceinline__ uint64_t make_desc(uint32_t addr16, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(addr16), "r"(hi));
    return d;
}
__device__ __forceinline__ uint32_t idesc_nvf4(int n) {
    // a/b format E2M1 (1), K-major both, N >> 3, scale format UE4M3 (0), M = 128 (>> 4), K = 64
    return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
}

__device__ __forceinline__ void tc_timeout(const Workspace& ws, TcShared* sh) {
    atomicExch(&ws.counters[CNT_STATUS], VMOE_ERR_TIMEOUT);
    atomicExch(&sh->abort_flag, 1);
}


// host: cached cuTensorMapEncodeTiled of a 2-D byte tensor [rows, row_bytes], box [box_rows, 128 B], 128-byte swizzle
int get_encoder();
int make_map(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows);
int make_sf_map(CUtensorMap* map, const void* base, uint64_t atoms);   // scale atoms [atoms, 512 B], box = 4 atoms
int tc_sm_count();

}  // namespace vmoe
