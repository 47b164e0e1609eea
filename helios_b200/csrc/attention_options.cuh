// What an attention kernel may be asked for beyond scaled dot products, a causal mask and a
// window; everything off in a zeroed struct.
//   slopes  float [heads]: score - slopes[h] * (query position - key position)
//   sink    the softmax has a key of score 0 that carries no value: the weights are
//           exp(s_j) / (1 + sum_j exp(s_j))
//   gate    [tokens, >= heads], rows gate_stride elements apart: head h's output at token t
//           is multiplied by sigmoid(gate[t, h])
#pragma once
#include "common.cuh"

struct AttnOptions {
  const float* slopes;
  const __nv_bfloat16* gate;
  int gate_stride;
  int sink;
};

// One output value from an accumulator `acc` and the row's maximum M (log2 domain) and sum L,
// both relative to M: the sink joins the sum as exp2(0 - M'), M' = max(M, 0); then the gate.
// With no sink and a factor of 1 this is acc / L, bit for bit.
__device__ __forceinline__ float attn_finish(float acc, float M, float L, int sink, float gate_factor) {
  if (sink) {
    const float Mn = fmaxf(M, 0.f);
    const float f = exp2f(M - Mn);
    acc *= f;
    L = L * f + exp2f(-Mn);
  }
  return acc / L * gate_factor;
}

__device__ __forceinline__ float attn_gate_factor(const AttnOptions& opt, size_t token, int head) {
  if (opt.gate == nullptr) return 1.f;
  const float g = __bfloat162float(opt.gate[token * (size_t)opt.gate_stride + head]);
  return 1.f / (1.f + __expf(-g));
}

// What a decode kernel that takes the step's q | k | v rows straight from the projection does
// to them on the way in, beside (or instead of) a rotation: q and k heads divided by their
// root mean square (eps inside the root) and multiplied by a weight per channel (wq, wk: float
// [head_dim], one for all heads; null: no norm), the query also by
// 1 + coef * ln(floor((position + 1) / every) + 1) (every 0: no such factor).
struct QkPrepare {
  const float* wq;
  const float* wk;
  float eps;
  float coef;
  int every;
};
