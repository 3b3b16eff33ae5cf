// Launchers of the NVFP4 kernels (mgbs_nvfp4.cu), called by the MLP scorer's host code.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgbs {

struct Nvfp4HeadArgs {
  const uint32_t* count_dev;  // rows to process (device value)
  int64_t row_limit;
  int32_t n_total;            // hidden units of layer 2 (multiple of 256)
  int32_t k_total;            // reduction length (multiple of 256)
  const uint8_t* sfa;         // block factors of the activations, [row tile][K-block][step][512 B]
  const uint8_t* sfb;         // block factors of the weights, [chunk of 256 rows][K-block][group of 128 rows][step][512 B]
  const float* bias;          // [n_total]
  const float* col_scale;     // [n_total]: product of the two tensor scales (per output channel)
  const float* w_out;         // [n_total] weights of the scalar head
  float* out_q;               // [rows]
  int32_t accumulate_q;
  int* err;
};

int nvfp4_prepare();
int launch_quant_h1_nvfp4(const uint8_t* h1_e4m3, const uint32_t* count_dev, int64_t row_limit, int K, float in_scale,
                          float inv_global, uint8_t* out_fp4, uint8_t* out_sf, int sms, cudaStream_t st);
// wide = 1: 256-column accumulator tiles with the factor copies on a thread of their own (K = 1024 only); 0: 128-column
// tiles with two accumulators
// tmB: weight rows in boxes of 128 (the 128-column kernel); tmBw: in boxes of 256 (the wide kernel)
int launch_head_nvfp4(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmBw, const Nvfp4HeadArgs& g, int sms,
                      cudaStream_t st, int wide);

}  // namespace mgbs
