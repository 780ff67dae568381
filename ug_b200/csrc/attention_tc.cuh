// Interface of the tcgen05 / TMEM causal prefill attention translation unit.
#pragma once
#include <cuda_bf16.h>

#include "ugb_internal.h"

// out[b, i, head, :] = softmax_j(scale * q[b, i, head, :] . k[b, kvh, j, :]) v[b, kvh, j, :] over the cached
// positions j <= pos0 + i, for i in [0, t).  q bf16 [batch, t, n_heads, 64] (rope applied), caches bf16
// [batch, n_kv, t_max, 64], out bf16 [batch, t, n_heads * 64].  All base pointers 16-byte aligned.
// dynamic != 0: the persistent CTAs draw their work items from the device's counter (longest first);
// 0: the items are dealt round-robin.
int32_t ugb_prefill_attention_tc(ugb_device *dev, const __nv_bfloat16 *q, const __nv_bfloat16 *kcache,
                                 const __nv_bfloat16 *vcache, __nv_bfloat16 *out, int batch, int t, int pos0,
                                 int n_heads, int n_kv, int t_max, float scale, int dynamic);
