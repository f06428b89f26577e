/* Private to development builds (-DVMOE_PROFILE): not installed, not part of the C ABI of include/vmoe.h. */
#ifndef VMOE_DEBUG_H_
#define VMOE_DEBUG_H_
#ifdef __cplusplus
extern "C" {
#endif
/* Cycle counters per warp role of the token-major tensor-core kernels, summed over CTAs since the previous
 * call: [0] MMA warp waiting for data, [1] for the accumulator, [2] issuing; [3] epilogue waiting, [4] working;
 * [5] producer waiting for a ring slot; [6] items; [7] stages; [8..10] epilogue: TMEM loads, arithmetic, stores.
 * Synchronises the device. */
int vmoe_debug_read_profile(unsigned long long* out12);
/* The same for the CTA-pair kernels: [0] MMA warp waiting for its own stage, [1] for the odd CTA's stage, [2] for the
 * accumulator, [3] issuing; [4] / [5] producer of the even / odd CTA waiting for a slot; [6] / [7] one epilogue warp
 * waiting / working; [8] items; [9] relay warp waiting; [10] MMA warp in total. */
int vmoe_debug_read_pair_profile(unsigned long long* out16);
#ifdef __cplusplus
}
#endif
#endif
