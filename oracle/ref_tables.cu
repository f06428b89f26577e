// Test infrastructure, not part of the product: a C entry point around the reference's own host-side
// permutation by expert (build_group_tables, fused-moe/csrc/verdict_fused_grouped.cu:655-691 of the
// reference project: std::stable_sort of the token-major pairs by expert id, expert list, token counts,
// exclusive offsets, gather indices, scatter weights).  The reference file is compiled where it lies (given
// with -I at build time, see build_ref.py); none of its text is copied here.  Its kernel is compiled too
// but never launched, so the library works on a machine without a GPU.
#define main verdict_grouped_main
#include "fused-moe/csrc/verdict_fused_grouped.cu"
#undef main

extern "C" {

// ids: [M, 10] int32 (the reference's routing rows are ten wide; columns >= topk are ignored).
// Outputs sized by the caller: expert_list / count [<= M*topk], offset [<= M*topk + 1], gather_idx /
// scatter_w [M*topk].  Returns the number of groups (experts that received at least one pair).
int ref_build_group_tables(const int* ids, int M, int topk, float weight, int* expert_list, int* count,
                           int* offset, int* gather_idx, float* scatter_w) {
    const GroupTables gt = build_group_tables(M, topk, reinterpret_cast<const int(*)[10]>(ids), weight);
    for (int g = 0; g < gt.num_groups; ++g) { expert_list[g] = gt.expert_list[g]; count[g] = gt.expert_token_count[g]; }
    for (int g = 0; g <= gt.num_groups; ++g) offset[g] = gt.expert_token_offset[g];
    for (int i = 0; i < gt.total_pairs; ++i) { gather_idx[i] = gt.gather_idx[i]; scatter_w[i] = gt.scatter_weights[i]; }
    return gt.num_groups;
}

}  // extern "C"
