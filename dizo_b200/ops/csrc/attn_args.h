// Launch description shared by the attention forward kernels (attn_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace dz {

struct AttnArgs {
  int B, L, H, hd;
  int n_prefix;
  long long ld_out;          // row stride of the context output (elements)
  __nv_bfloat16* out;        // [B*L, ld_out], head h at columns [h*hd, (h+1)*hd)
  const int* pad_left;       // [B] or null
  float* lse;                // [B, H, L] or null: log2-domain log-sum-exp of every query row
  float scale_log2;          // softmax scale * log2(e)
  int q_col0, k_col0, v_col0;  // first column of the Q / K / V sections inside the QKV rows
  uint32_t* err;
};

}  // namespace dz
