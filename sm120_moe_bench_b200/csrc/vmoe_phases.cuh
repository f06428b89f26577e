// Device functions of the small stages of the layer (router, permutation tables, permuting activation
// quantiser, combine), shared by their stand-alone kernels.
//
// Router semantics: fused-moe/csrc/megakernel_v1.cu:491-537 of the reference; permutation:
// fused-moe/csrc/verdict_fused_grouped.cu:655-691; quantiser: fused-moe/csrc/verdict_fused_cooperative_tma_ext.cu
// :249-279; combine: the same file, :549-563.
#pragma once
#include "vmoe_common.cuh"

namespace vmoe {

// One warp routes one token: p = the warp's E floats of shared memory, l = the token's logits.
// fp32 softmax, T rounds of arg-max under (probability desc, expert id asc), renormalise.
// A row with a NaN or +inf logit has only NaN probabilities (the reference then leaves its ids at -1,
// fused-moe/csrc/megakernel_v1.cu:516-528); here a NaN probability counts as 0 in the selection, so the ids
// are always distinct and inside [0, E) and the row's weights come out NaN (0 / 0).
__device__ __forceinline__ void route_token(const float* l, float* p, int E, int T, int lane,
                                            int32_t* ids_out, float* w_out) {
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) { float v = l[e]; p[e] = v; mx = fmaxf(mx, v); }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) { float v = expf(p[e] - mx); p[e] = v; sum += v; }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) { const float v = p[e] * inv; p[e] = (v == v) ? v : 0.0f; }
    __syncwarp();

    // Every lane keeps the best of its own (strided) entries; a round is two warp reductions -- the largest value
    // (probabilities are >= 0, so their bit patterns order like unsigned integers), then the lowest expert id
    // among the lanes that hold it -- and only the winning lane rescans its entries.
    auto local_best = [&](float& bv, int& bi) {
        bv = -1.0f; bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) { const float v = p[e]; if (v > bv) { bv = v; bi = e; } }
    };
    float bv; int bi;
    local_best(bv, bi);
    float sel_w = 0.f; int sel_id = 0; float wsum = 0.f;   // lane j keeps the j-th selection
    for (int j = 0; j < T; ++j) {
        const unsigned key = bv >= 0.0f ? __float_as_uint(bv) + 1u : 0u;
        const unsigned top = __reduce_max_sync(0xffffffffu, key);
        const unsigned win = __reduce_min_sync(0xffffffffu, key == top ? (unsigned)bi : 0x7fffffffu);
        const float wv = top ? __uint_as_float(top - 1u) : 0.0f;
        if (lane == j) { sel_w = wv; sel_id = (int)win; }
        wsum += wv;                              // same value in every lane, rank order
        if (win < (unsigned)E && (int)(win & 31u) == lane) {       // taken (T <= E: an untaken entry >= 0 always exists)
            p[win] = -2.0f;
            local_best(bv, bi);
        }
    }
    const float winv = 1.0f / wsum;
    if (lane < T) {
        ids_out[lane] = min(max(sel_id, 0), E - 1);
        w_out[lane] = sel_w * winv;
    }
}

// ---------------------------------------------------------------------------------
// Permutation tables (see vmoe_route.cu for the description of the phases)
// ---------------------------------------------------------------------------------
struct TableArgs {
    const int32_t* ids; const float* w; const int32_t* expert_map;
    int M, T, E, has_shared, words;   // words = ceil(M / 32)
    int num_global;                   // range of the ids (length of expert_map when there is one)
    int tiles_d;                      // column tiles of the down projection (hidden / 128); 0 = no dependency counters
    int tc_cap;                       // tokens per tensor-core unit
    int gemv_units;                   // also emit the 4-token work units of the CUDA-core path
    Workspace ws;
};

// Local expert of pair p, -1 when the pair is dropped: its expert lives on another GPU, or its id is outside
// [0, num_global) -- caller-supplied ids are never used as an index unchecked; an id past the range also
// sets VMOE_ERR_LIMIT in the status word (negative ids are the framework's "no expert" marker and drop silently).
__device__ __forceinline__ int local_expert(const TableArgs& a, int p) {
    int e = a.ids[p];
    if ((unsigned)e >= (unsigned)a.num_global) {
        if (e >= 0 && a.ws.counters) atomicExch(&a.ws.counters[CNT_STATUS], VMOE_ERR_LIMIT);
        return -1;
    }
    if (a.expert_map) e = a.expert_map[e];
    return (e >= 0 && e < a.E) ? e : -1;
}

__device__ inline void phase_clear(const TableArgs& a, int tid, int nthr) {
    const int n = a.E * a.words;
    for (int i = tid; i < n; i += nthr) a.ws.bitmap[i] = 0u;
    if (tid < CNT_N && tid != CNT_STATUS) a.ws.counters[tid] = 0;
    // dependency counters of the fused weights-as-rows kernel
    if (a.ws.unit_done)
        for (int i = tid; i < a.ws.tc_unit_capacity; i += nthr) a.ws.unit_done[i] = 0;
    if (a.ws.token_done && a.tiles_d > 0 && a.M <= a.ws.small_tokens) {
        for (int i = tid; i < a.M * a.tiles_d; i += nthr) a.ws.token_done[i] = 0;
        for (int i = tid; i < a.M; i += nthr) a.ws.token_expect[i] = 0;
    }
}
__device__ inline void phase_mark(const TableArgs& a, int tid, int nthr) {
    const int P = a.M * a.T;
    for (int p = tid; p < P; p += nthr) {
        const int e = local_expert(a, p);
        if (e >= 0) { const int m = p / a.T; atomicOr(&a.ws.bitmap[(size_t)e * a.words + (m >> 5)], 1u << (m & 31)); }
    }
}
// Running popcount per bitmap word and the pair count per expert.  A warp takes 32 / wp experts at a
// time (wp = words rounded up to a power of two) with a segmented shuffle scan over each expert's
// words; experts with more than 32 words are walked 32 words at a time by a whole warp.
__device__ inline void phase_count(const TableArgs& a, int warp, int nwarps, int lane, int32_t* s_count) {
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
__device__ inline void phase_scan(const TableArgs& a, int tid, int nthr, const int32_t* s_count, int32_t* s_scan) {
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
                    if (t < a.ws.tc_unit_capacity) a.ws.tc_units[t] = make_int4(e, c + s, nt, tc_box(nt));
                    else a.ws.counters[CNT_STATUS] = VMOE_ERR_LIMIT;     // more units than the workspace was sized for
                    ++t;
                }
            }
            c += cnt;
        }
    }
}
__device__ inline void phase_place(const TableArgs& a, int tid, int nthr) {
    const int P = a.M * a.T;
    const bool count_rows = a.ws.token_done && a.tiles_d > 0 && a.M <= a.ws.small_tokens;
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
            if (count_rows) atomicAdd(&a.ws.token_expect[m], 1);      // rows the token's combine waits for
        }
        a.ws.pair_slot[p] = slot;
    }
    if (a.has_shared) {
        const int base = a.ws.expert_offsets[a.E];
        for (int m = tid; m < a.M; m += nthr) {
            a.ws.sorted_pair[base + m] = P + m;
            a.ws.gather_idx[base + m] = m;
            a.ws.scatter_weights[base + m] = 1.0f;
            if (count_rows) atomicAdd(&a.ws.token_expect[m], 1);
        }
    }
}


// The activation quantiser on one block of 16 bf16 values (…tma_ext.cu:249-279: amax / 6 floored at 1e-30 -> E4M3,
// round to nearest even, saturating -> decoded scale floored at 1e-30 -> e2m1(x / scale), even element in the low nibble).
__device__ __forceinline__ void quantize_block16(const __nv_bfloat16* h, float (&v)[SF_BLOCK], uint32_t& lo, uint32_t& hi, uint8_t& sb) {
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < SF_BLOCK; ++i) { v[i] = __bfloat162float(h[i]); amax = fmaxf(amax, fabsf(v[i])); }
    sb = e4m3_encode(fmaxf(amax / 6.0f, 1e-30f));
    float scale = e4m3_decode(sb);
    if (scale < 1e-30f) scale = 1e-30f;
    const ScaleDivider div_scale(scale);
    lo = 0; hi = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) lo |= e2m1_encode(div_scale(v[i])) << (4 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i) hi |= e2m1_encode(div_scale(v[8 + i])) << (4 * i);
}

// Permuting activation quantiser for one 16-element block b of the token-major activations: quantise
// (same arithmetic as quantize_kernel) and write the codes to the token-order copy and to every sorted slot
// of the token, the block scale into the per-unit atom layout of the tensor-core B operand.
template <bool BATCHED>
__device__ __forceinline__ void permute_quantize_block(long long b, const __nv_bfloat16* __restrict__ x, int M, int K, int T, int E,
                                                       int has_shared, int tc_cap, const int32_t* topk_ids,
                                                       const int32_t* expert_map, const Workspace& ws,
                                                       const uint8_t* pre_q = nullptr, const uint8_t* pre_sf = nullptr) {
    const int bpr = K / SF_BLOCK;
    const int cap_shift = 31 - __clz(tc_cap);
    const int m = (int)(b / bpr), kb = (int)(b % bpr);
    // the row's data is requested first: its latency then overlaps the table reads below
    uint4 raw[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
    uint2 pre_c = make_uint2(0, 0); uint8_t pre_s = 0;
    if (pre_q) { pre_c = reinterpret_cast<const uint2*>(pre_q)[b]; pre_s = pre_sf[b]; }
    else { const uint4* src = reinterpret_cast<const uint4*>(x + b * SF_BLOCK); raw[0] = src[0]; raw[1] = src[1]; }
    // Destinations of the row: one per routed pair plus the shared expert.  BATCHED (small launches, bound by
    // load latency): all table reads of one level are issued together, three dependent round trips for the
    // whole row instead of four per pair.  Large launches walk the pairs one by one with fewer registers.
    constexpr int MAXJ = MAX_TOPK + 1;
    int slot[BATCHED ? MAXJ : 1], ex[BATCHED ? MAXJ : 1], off[BATCHED ? MAXJ : 1], ub[BATCHED ? MAXJ : 1];
    if (BATCHED) {
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
            slot[j] = -1; ex[j] = -1;
            if (j < T) { slot[j] = ws.pair_slot[m * T + j]; ex[j] = topk_ids[m * T + j]; }
        }
        const int shared_base = has_shared ? ws.expert_offsets[E] : 0;
        if (expert_map) {
#pragma unroll
            for (int j = 0; j < MAXJ; ++j) if (j < T && slot[j] >= 0) ex[j] = expert_map[ex[j]];
        }
#pragma unroll
        for (int j = 0; j < MAXJ; ++j) {
            if (j == T && has_shared) { slot[j] = shared_base + m; ex[j] = E; }
            off[j] = 0; ub[j] = 0;
            if (slot[j] >= 0) { off[j] = ws.expert_offsets[ex[j]]; ub[j] = ws.tc_unit_base[ex[j]]; }
        }
    }
    uint32_t lo = 0, hi = 0;
    uint8_t sb;
    if (pre_q) {
        // the row arrives quantised (a previous layer's fused RMSNorm + quantise epilogue)
        lo = pre_c.x; hi = pre_c.y; sb = pre_s;
    } else {
        const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(raw);
        float v[SF_BLOCK];
        quantize_block16(h, v, lo, hi, sb);
    }
    // token-order copy (stage-wise checks and the GEMV path read it)
    reinterpret_cast<uint2*>(ws.act_q)[b] = make_uint2(lo, hi);
    ws.act_sf[b] = sb;
    auto put = [&](int sl, int o, int u0) {
        const int rank = sl - o;
        const int unit = u0 + (rank >> cap_shift);          // tc_cap is 16, 64 or 128
        const int r = rank & (tc_cap - 1);
        reinterpret_cast<uint2*>(ws.act_q_sorted + (size_t)sl * (K / 2))[kb] = make_uint2(lo, hi);
        ws.act_sf_atoms[((size_t)unit * (K / 64) + (kb >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb & 3)] = sb;
    };
    if (BATCHED) {
#pragma unroll
        for (int j = 0; j < MAXJ; ++j)
            if (slot[j] >= 0) put(slot[j], off[j], ub[j]);
    } else {
        for (int j = 0; j <= T; ++j) {
            int e, sl;
            if (j < T) {
                sl = ws.pair_slot[m * T + j];
                if (sl < 0) continue;
                e = topk_ids[m * T + j];
                if (expert_map) e = expert_map[e];
            } else {
                if (!has_shared) break;
                e = E;
                sl = ws.expert_offsets[E] + m;
            }
            put(sl, ws.expert_offsets[e], ws.tc_unit_base[e]);
        }
    }
}

// Expert parallelism: NB 16-element blocks (block b = received row b / bpr of the dense list, k-block b % bpr; b < 0 =
// none) go to their sorted slots + scale atoms; a block with k-block 0 also records where its slot's output row goes:
// the row of the pair in its owner's combine area.  Row i of the dense list = source s, position i - src_base[s].
// The table reads of all NB blocks are issued level by level (three dependent round trips for the batch, not per block).
template <int NB>
__device__ __forceinline__ void ep_permute_blocks(const TcEpPermute& e, const long long (&b)[NB], int K, int tc_cap, const Workspace& ws) {
    const int bpr = K / SF_BLOCK;
    const int cap_shift = 31 - __clz(tc_cap);                     // tc_cap is 16 or 128
    int row_i[NB], kb[NB], slot[NB], ex[NB], src[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        slot[n] = -1; ex[n] = 0; row_i[n] = 0; kb[n] = 0;
        if (b[n] >= 0) { row_i[n] = (int)(b[n] / bpr); kb[n] = (int)(b[n] % bpr); slot[n] = ws.pair_slot[row_i[n]]; ex[n] = e.flat_ids[row_i[n]]; }
    }
    uint2 q[NB]; uint8_t sb[NB]; int off[NB], ub[NB]; size_t row[NB];
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        src[n] = 0; row[n] = 0; off[n] = 0; ub[n] = 0; q[n] = make_uint2(0, 0); sb[n] = 0;
        if (slot[n] < 0) continue;
        while (src[n] + 1 < e.world && row_i[n] >= e.src_base[src[n] + 1]) ++src[n];
        row[n] = (size_t)src[n] * e.capacity + (row_i[n] - e.src_base[src[n]]);
        q[n] = reinterpret_cast<const uint2*>(e.recv_q + row[n] * (K / 2))[kb[n]];
        sb[n] = (e.recv_sf + row[n] * (K / 16))[kb[n]];
        off[n] = ws.expert_offsets[ex[n]]; ub[n] = ws.tc_unit_base[ex[n]];
    }
#pragma unroll
    for (int n = 0; n < NB; ++n) {
        if (slot[n] < 0) continue;
        const int rank_in_e = slot[n] - off[n];
        const int unit = ub[n] + (rank_in_e >> cap_shift);
        const int r = rank_in_e & (tc_cap - 1);
        reinterpret_cast<uint2*>(ws.act_q_sorted + (size_t)slot[n] * (K / 2))[kb[n]] = q[n];
        if (unit < ws.tc_unit_capacity)
            ws.act_sf_atoms[((size_t)unit * (K / 64) + (kb[n] >> 2)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kb[n] & 3)] = sb[n];
        if (kb[n] == 0) e.row_dst[slot[n]] = e.comb[src[n]] + (size_t)e.recv_meta[row[n]].y * K;     // row of the pair in its owner's slab
    }
}
// out[m, 4c .. 4c+3] = bf16( sum_j pair_out[slot(m, j), :]  (ascending j, fp32)  + shared row ) [+ residual],
// element i = m * (K / 4) + c.  BATCHED: slot numbers and then all rows requested at once (small launches).
// Four consecutive values of one per-pair row: fp32 as stored, or bf16 widened (ROWS16).
template <bool ROWS16>
__device__ __forceinline__ float4 pair_row_load(const float* pair_out, size_t slot, int K, int c) {
    if (ROWS16) {
        const uint2 u = __ldcg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(pair_out) + slot * K) + c);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&u.x), b = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        return make_float4(__bfloat162float(a.x), __bfloat162float(a.y), __bfloat162float(b.x), __bfloat162float(b.y));
    }
    return __ldcg(reinterpret_cast<const float4*>(pair_out + slot * K) + c);       // L2: rows written by other SMs
}
template <bool BATCHED, bool ROWS16 = false>
__device__ __forceinline__ uint2 combine_value(long long i, const float* pair_out, const int32_t* pair_slot,
                                               const int32_t* expert_offsets, int K, int T, int E, int has_shared,
                                               const __nv_bfloat16* residual) {
    const int k4 = K / 4;
    const int m = (int)(i / k4), c = (int)(i % k4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (BATCHED) {
        int slot[MAX_TOPK + 1];
#pragma unroll
        for (int j = 0; j < MAX_TOPK; ++j) slot[j] = (j < T) ? pair_slot[m * T + j] : -1;
        slot[MAX_TOPK] = has_shared ? expert_offsets[E] + m : -1;
        float4 v[MAX_TOPK + 1];
#pragma unroll
        for (int j = 0; j <= MAX_TOPK; ++j)
            if (slot[j] >= 0) v[j] = pair_row_load<ROWS16>(pair_out, (size_t)slot[j], K, c);
#pragma unroll
        for (int j = 0; j <= MAX_TOPK; ++j)        // ascending pair order, shared expert last
            if (slot[j] >= 0) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    } else {
        for (int j = 0; j < T; ++j) {
            const int slot = pair_slot[m * T + j];
            if (slot >= 0) {
                const float4 v = pair_row_load<ROWS16>(pair_out, (size_t)slot, K, c);
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        }
        if (has_shared) {
            const int slot = expert_offsets[E] + m;
            const float4 v = pair_row_load<ROWS16>(pair_out, (size_t)slot, K, c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
    if (residual) {
        // x + moe(x) with the layer output rounded to bf16 first: the same bits as a separate bf16 add
        const uint2 r = reinterpret_cast<const uint2*>(residual + (size_t)m * K)[c];
        const __nv_bfloat162 r0 = *reinterpret_cast<const __nv_bfloat162*>(&r.x), r1 = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        lo = __floats2bfloat162_rn(__bfloat162float(r0.x) + __bfloat162float(lo.x), __bfloat162float(r0.y) + __bfloat162float(lo.y));
        hi = __floats2bfloat162_rn(__bfloat162float(r1.x) + __bfloat162float(hi.x), __bfloat162float(r1.y) + __bfloat162float(hi.y));
    }
    uint2 o; o.x = *reinterpret_cast<uint32_t*>(&lo); o.y = *reinterpret_cast<uint32_t*>(&hi);
    return o;                       // four bf16 values
}
template <bool BATCHED, bool ROWS16 = false>
__device__ __forceinline__ void combine_element(long long i, const float* pair_out, const int32_t* pair_slot,
                                                const int32_t* expert_offsets, int M, int K, int T, int E, int has_shared,
                                                const __nv_bfloat16* residual, __nv_bfloat16* out) {
    (void)M;
    reinterpret_cast<uint2*>(out)[i] = combine_value<BATCHED, ROWS16>(i, pair_out, pair_slot, expert_offsets, K, T, E, has_shared, residual);
}

}  // namespace vmoe
