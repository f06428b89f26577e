// Test infrastructure, not part of the product: C entry points around the reference's own host-side
// C++ reference (fused-moe/csrc/verdict_fused_independent.cu of the reference project: h_e4m3fn_decode :50-55,
// h_e4m3fn_encode :57-71, h_e4m3fn_encode_ceil :73-84, quantize_to_nvfp4_e4m3 :474-496,
// dequant_fp4_e4m3 :498-504, host_quantized_reference_single :509-564).  The reference file is compiled
// where it lies (given with -I at build time, see build_ref.py); none of its text is copied here.  Its
// kernels are compiled too but never launched: only the host functions are called, so the library
// works on a machine without a GPU.
#define main verdict_reference_main
#include "fused-moe/csrc/verdict_fused_independent.cu"
#undef main

extern "C" {

int ref_hidden(void) { return HIDDEN; }
float ref_e4m3_decode(unsigned char x) { return h_e4m3fn_decode(x); }
unsigned char ref_e4m3_encode(float v) { return h_e4m3fn_encode(v); }
unsigned char ref_e4m3_encode_ceil(float v) { return h_e4m3fn_encode_ceil(v); }
float ref_silu(float x) { return host_silu(x); }
void ref_quantize(const float* data, int numel, unsigned char* packed, unsigned char* sf) {
    quantize_to_nvfp4_e4m3(data, numel, packed, sf);
}
float ref_dequant(const unsigned char* packed, const unsigned char* sf, int idx) { return dequant_fp4_e4m3(packed, sf, idx); }
// one token (already quantised, HIDDEN elements) through `na` experts with weights `ewts`; out: HIDDEN floats
void ref_layer_single(const unsigned char* ifp4, const unsigned char* isf, const unsigned char* w1f, const unsigned char* w1s,
                      const unsigned char* w2f, const unsigned char* w2s, const int* eids, const float* ewts, float* out,
                      int na, int n_half) {
    host_quantized_reference_single(ifp4, isf, w1f, w1s, w2f, w2s, eids, ewts, out, na, n_half);
}

}  // extern "C"
