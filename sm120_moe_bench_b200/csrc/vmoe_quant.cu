// bf16 -> NVFP4 activation quantiser, the NVFP4 -> f32 decoder and the deterministic combine.
//
// Quantiser arithmetic: fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu:249-279 of the
// reference (per 16 consecutive elements: amax / 6 floored at 1e-30 -> E4M3 RNE saturating ->
// decoded scale floored at 1e-30 -> e2m1(x / scale), even element in the low nibble).
// Combine: …tma_ext.cu:549-563 (fp32 sum over a token's pairs in ascending pair order -> bf16).
#include "vmoe_common.cuh"
#include "vmoe_phases.cuh"

namespace vmoe {

// One thread per 16-element block: 32 bytes in, 8 + 1 bytes out.
__global__ void __launch_bounds__(256)
quantize_kernel(const __nv_bfloat16* __restrict__ x, long long nblocks, int blocks_per_row,
                uint8_t* __restrict__ packed, uint8_t* __restrict__ sf) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + b * SF_BLOCK);
    uint4 raw[2] = {src[0], src[1]};
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(raw);
    float v[SF_BLOCK];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < SF_BLOCK; ++i) { v[i] = __bfloat162float(h[i]); amax = fmaxf(amax, fabsf(v[i])); }
    const float target = fmaxf(amax / 6.0f, 1e-30f);
    const uint8_t sb = e4m3_encode(target);
    float scale = e4m3_decode(sb);
    if (scale < 1e-30f) scale = 1e-30f;
    uint32_t lo = 0, hi = 0;
    const ScaleDivider div_scale(scale);
#pragma unroll
    for (int i = 0; i < 8; ++i)  lo |= e2m1_encode(div_scale(v[i])) << (4 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i)  hi |= e2m1_encode(div_scale(v[8 + i])) << (4 * i);
    reinterpret_cast<uint2*>(packed)[b] = make_uint2(lo, hi);
    sf[b] = sb;
    (void)blocks_per_row;
}

int launch_quantize(const __nv_bfloat16* x, int rows, int K, uint8_t* packed, uint8_t* sf, cudaStream_t st) {
    const long long nblocks = (long long)rows * (K / SF_BLOCK);
    if (nblocks == 0) return VMOE_OK;
    quantize_kernel<<<(unsigned)((nblocks + 255) / 256), 256, 0, st>>>(x, nblocks, K / SF_BLOCK, packed, sf);
    return cuda_status(cudaGetLastError());
}

__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ sf,
                  const float* __restrict__ gs, long long nblocks, int blocks_per_row,
                  long long rows_per_scale, float* __restrict__ out) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const uint2 c = reinterpret_cast<const uint2*>(packed)[b];
    const float s = e4m3_decode(sf[b]);
    const float g = gs ? gs[(b / blocks_per_row) / rows_per_scale] : 1.0f;
    float* o = out + b * SF_BLOCK;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = e2m1_decode((c.x >> (4 * i)) & 0xF) * s * g;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[8 + i] = e2m1_decode((c.y >> (4 * i)) & 0xF) * s * g;
}

int launch_dequantize(const uint8_t* packed, const uint8_t* sf, const float* gs, int64_t rows, int K,
                      int64_t rows_per_scale, float* out, cudaStream_t st) {
    const long long nblocks = (long long)rows * (K / SF_BLOCK);
    if (nblocks == 0) return VMOE_OK;
    dequantize_kernel<<<(unsigned)((nblocks + 255) / 256), 256, 0, st>>>(
        packed, sf, gs, nblocks, K / SF_BLOCK, rows_per_scale > 0 ? rows_per_scale : 1, out);
    return cuda_status(cudaGetLastError());
}

// out[m, :] = bf16( sum_j pair_out[slot(m, j), :]  (ascending j, fp32)  + shared row )
// one thread per 4 consecutive columns.  BATCHED (small launches, bound by load latency): the slot numbers and
// then all rows of a token are requested at once; otherwise (large launches, bound by bandwidth) row by row.
template <bool BATCHED, bool ROWS16>
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ pair_out, const int32_t* __restrict__ pair_slot,
               const int32_t* __restrict__ expert_offsets, int M, int K, int T, int E, int has_shared,
               const __nv_bfloat16* residual, __nv_bfloat16* out) {      // residual may alias out
    pdl_begin();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)M * (K / 4)) return;
    combine_element<BATCHED, ROWS16>(i, pair_out, pair_slot, expert_offsets, M, K, T, E, has_shared, residual, out);
}

int launch_combine(const vmoe_shape& s, int M, const Workspace& ws, __nv_bfloat16* out, cudaStream_t st,
                   const __nv_bfloat16* residual) {
    const long long n = (long long)M * (s.hidden / 4);
    if (n == 0) return VMOE_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (ws.pair_rows_bf16)
        launch_pdl(combine_kernel<false, true>, blocks, 256u, 0, st,
            ws.pair_out, ws.pair_slot, ws.expert_offsets, M, s.hidden, s.topk, s.num_experts, s.has_shared, residual, out);
    else if (blocks <= 1024)
        launch_pdl(combine_kernel<true, false>, blocks, 256u, 0, st,
            ws.pair_out, ws.pair_slot, ws.expert_offsets, M, s.hidden, s.topk, s.num_experts, s.has_shared, residual, out);
    else
        launch_pdl(combine_kernel<false, false>, blocks, 256u, 0, st,
            ws.pair_out, ws.pair_slot, ws.expert_offsets, M, s.hidden, s.topk, s.num_experts, s.has_shared, residual, out);
    return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------------
// RMSNorm + NVFP4 quantisation of a row, either of a given matrix or of the combine's result (fused behind the
// combine: the row is summed, the residual added, written, normalised and quantised in one pass over it).
// Follows rmsnorm_parallel + rmsnorm_apply_and_quantize (fused-moe/csrc/megakernel_v1.cu:257-352): sum of squares
// over the row, scale by 1 / sqrt(mean + eps) and by gamma, quantise per 16 elements.  The reference keeps the
// residual stream in f32 and uses rsqrtf; here the stream is bf16 (what the operator's caller holds), the
// normalised row is rounded to bf16 before it is quantised (the activation quantiser's input type) and the
// reciprocal square root is IEEE (1 / sqrtf), so the result is reproducible bit for bit.
// One CTA of 256 threads per row; a thread owns the 16-element blocks b = tid, tid + 256, ...  Order of the sum
// of squares (part of the definition, restated by the oracle): per thread in element order across its blocks, then
// the warp's xor tree (16, 8, 4, 2, 1), then the eight warp sums in warp order.
// ---------------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;

template <bool FROM_COMBINE>
__global__ void __launch_bounds__(NORM_THREADS)
norm_quant_kernel(const __nv_bfloat16* x, const float* __restrict__ pair_out, const int32_t* __restrict__ pair_slot,
                  const int32_t* __restrict__ expert_offsets, int K, int T, int E, int has_shared,
                  const __nv_bfloat16* residual, __nv_bfloat16* out,          // FROM_COMBINE: the combined row goes here
                  const float* __restrict__ gamma, float eps, __nv_bfloat16* normed, uint8_t* packed, uint8_t* sf) {
    extern __shared__ float s_row[];                 // [K] the row as f32
    __shared__ float s_warp[NORM_THREADS / 32];
    pdl_begin();
    const int m = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nblk = K / SF_BLOCK;
    float ss = 0.f;
    for (int b = tid; b < nblk; b += NORM_THREADS) {
        uint2 q[4];
        if (FROM_COMBINE) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                q[i] = combine_value<true>((long long)m * (K / 4) + b * 4 + i, pair_out, pair_slot, expert_offsets, K, T, E, has_shared, residual);
                reinterpret_cast<uint2*>(out + (size_t)m * K)[b * 4 + i] = q[i];
            }
        } else {
            const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)m * K + (size_t)b * SF_BLOCK);
            const uint4 r0 = src[0], r1 = src[1];
            q[0] = make_uint2(r0.x, r0.y); q[1] = make_uint2(r0.z, r0.w); q[2] = make_uint2(r1.x, r1.y); q[3] = make_uint2(r1.z, r1.w);
        }
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(q);
#pragma unroll
        for (int i = 0; i < SF_BLOCK; ++i) {
            const float v = __bfloat162float(h[i]);
            s_row[b * SF_BLOCK + i] = v;
            ss = fmaf(v, v, ss);
        }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) s_warp[warp] = ss;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < NORM_THREADS / 32; ++w) total += s_warp[w];
    const float rms = 1.0f / sqrtf(total / (float)K + eps);
    for (int b = tid; b < nblk; b += NORM_THREADS) {
        __align__(16) __nv_bfloat16 y[SF_BLOCK];
#pragma unroll
        for (int i = 0; i < SF_BLOCK; ++i) y[i] = __float2bfloat16_rn((s_row[b * SF_BLOCK + i] * rms) * gamma[b * SF_BLOCK + i]);
        if (normed) {
            uint4* dst = reinterpret_cast<uint4*>(normed + (size_t)m * K + (size_t)b * SF_BLOCK);
            dst[0] = reinterpret_cast<const uint4*>(y)[0]; dst[1] = reinterpret_cast<const uint4*>(y)[1];
        }
        float v[SF_BLOCK]; uint32_t lo, hi; uint8_t sb;
        quantize_block16(y, v, lo, hi, sb);
        reinterpret_cast<uint2*>(packed + (size_t)m * (K / 2))[b] = make_uint2(lo, hi);
        sf[(size_t)m * nblk + b] = sb;
    }
}

static int launch_norm(bool from_combine, const __nv_bfloat16* x, const vmoe_shape* s, const Workspace* ws, int rows, int K,
                       const __nv_bfloat16* residual, __nv_bfloat16* out, const float* gamma, float eps, __nv_bfloat16* normed,
                       uint8_t* packed, uint8_t* sf, cudaStream_t st) {
    if (rows == 0) return VMOE_OK;
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 200 * 1024) return VMOE_ERR_SHAPE;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(norm_quant_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(norm_quant_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_done = true;
    }
    if (from_combine)
        launch_pdl(norm_quant_kernel<true>, (unsigned)rows, (unsigned)NORM_THREADS, smem, st, x, ws->pair_out, ws->pair_slot,
                   ws->expert_offsets, K, s->topk, s->num_experts, s->has_shared, residual, out, gamma, eps, normed, packed, sf);
    else
        launch_pdl(norm_quant_kernel<false>, (unsigned)rows, (unsigned)NORM_THREADS, smem, st, x, (const float*)nullptr,
                   (const int32_t*)nullptr, (const int32_t*)nullptr, K, 0, 0, 0, (const __nv_bfloat16*)nullptr,
                   (__nv_bfloat16*)nullptr, gamma, eps, normed, packed, sf);
    return cuda_status(cudaGetLastError());
}

int launch_combine_norm(const vmoe_shape& s, int M, const Workspace& ws, __nv_bfloat16* out, cudaStream_t st,
                        const __nv_bfloat16* residual, const float* gamma, float eps, __nv_bfloat16* normed,
                        uint8_t* packed, uint8_t* sf) {
    return launch_norm(true, nullptr, &s, &ws, M, s.hidden, residual, out, gamma, eps, normed, packed, sf, st);
}
int launch_rmsnorm_quantize(const __nv_bfloat16* x, const float* gamma, float eps, int rows, int K, __nv_bfloat16* normed,
                            uint8_t* packed, uint8_t* sf, cudaStream_t st) {
    return launch_norm(false, x, nullptr, nullptr, rows, K, nullptr, nullptr, gamma, eps, normed, packed, sf, st);
}

// ---------------------------------------------------------------------------------
// Router projection: logits[m, e] = sum_k hidden[m, k] * gate_weight[e, k]  (f32 accumulation).
// Follows moe_gate_distributed (fused-moe/csrc/megakernel_v1.cu:455-489): one dot product per (token,
// expert).  One warp per expert and chunk of 8 tokens; a lane owns 8 consecutive k out of every 256 and
// sums them in ascending order, then the 32 lane sums go through an xor-shuffle tree: a fixed order,
// so the logits (and the routing that follows) are reproducible.
// ---------------------------------------------------------------------------------
constexpr int GEMV_TOK = 8;
__device__ __forceinline__ void load8(const float* p, float (&v)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(h[i]);
}
template <typename W>
__global__ void __launch_bounds__(256)
router_gemv_kernel(const __nv_bfloat16* __restrict__ x, const W* __restrict__ gw, int M, int K, int E, float* __restrict__ logits) {
    pdl_begin();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.x * 8 + warp;
    const int m0 = blockIdx.y * GEMV_TOK;
    if (e >= E) return;
    float acc[GEMV_TOK];
#pragma unroll
    for (int t = 0; t < GEMV_TOK; ++t) acc[t] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
        float w[8];
        load8(gw + (size_t)e * K + k, w);
#pragma unroll
        for (int t = 0; t < GEMV_TOK; ++t) {
            if (m0 + t < M) {
                float h[8];
                load8(x + (size_t)(m0 + t) * K + k, h);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[t] = fmaf(h[i], w[i], acc[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < GEMV_TOK; ++t) {
#pragma unroll
        for (int o = 16; o; o >>= 1) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], o);
        if (lane == 0 && m0 + t < M) logits[(size_t)(m0 + t) * E + e] = acc[t];
    }
}

int launch_router_gemv(const __nv_bfloat16* x, const void* gate_weight, int gate_dtype, int M, int K, int E,
                       float* logits, cudaStream_t st) {
    if (M == 0) return VMOE_OK;
    if (K % 256 || E <= 0 || (gate_dtype != 0 && gate_dtype != 1)) return VMOE_ERR_SHAPE;
    const dim3 grid((unsigned)((E + 7) / 8), (unsigned)((M + GEMV_TOK - 1) / GEMV_TOK));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t err;
    if (gate_dtype == 0)
        err = cudaLaunchKernelEx(&cfg, router_gemv_kernel<float>, x, static_cast<const float*>(gate_weight), M, K, E, logits);
    else
        err = cudaLaunchKernelEx(&cfg, router_gemv_kernel<__nv_bfloat16>, x, static_cast<const __nv_bfloat16*>(gate_weight), M, K, E, logits);
    return cuda_status(err != cudaSuccess ? err : cudaGetLastError());
}

}  // namespace vmoe
