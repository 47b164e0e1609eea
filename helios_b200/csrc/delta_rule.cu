// A recurrent mixer with a matrix state per head, written by the gated delta rule with one
// decay per key channel.  Per token and head (k, q unit vectors, q also times dk^-1/2):
//
//   S <- g (.) S            (g in (0,1)^dk scales the rows of S [dk, dv])
//   u  = beta (v - S^T k)
//   S <- S + k u^T
//   o  = S^T q              (the read-out sees this token's write)
//
// The columns of S never mix: a thread owns one column (dk values in registers) and walks
// the request's tokens in order, so a request's numbers do not depend on how its tokens
// were cut into steps or on the rest of the batch.  State, decays, gates, unit norms and
// the recurrence are float32.
//
// Kernels: `causal_conv_silu` (short causal convolution over time per channel + silu, the
// taps - 1 inputs before a step's first token taken from the request's slot),
// `causal_conv_state` (leaves the last taps - 1 inputs in the slot), `delta_rule` (the
// recurrence) and `gated_rmsnorm` (o / rms(o) * weight * sigmoid(gate) per head).
#include "common.cuh"

// ---------------------------------------------------------------- short convolution
// x [T, ld] (the first `channels` columns), w [channels, taps] (the last column is the
// current token's), conv state of a slot at state + slot * state_stride: [channels, taps - 1],
// oldest first.  out [T, channels].
template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ x, int ld,
                                        const float* __restrict__ w, const float* __restrict__ state,
                                        long state_stride, const int* __restrict__ seq_of_token,
                                        const int* __restrict__ cu_tokens,
                                        const int* __restrict__ slots, int n_tokens, int channels,
                                        int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_tokens * channels;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / channels), c = (int)(idx - (size_t)t * channels);
    const int s = seq_of_token[t];
    const int local = t - cu_tokens[s];
    const float* st = state + (size_t)slots[s] * state_stride + (size_t)c * (taps - 1);
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - (taps - 1) + j;
      const float v = src >= 0 ? to_float(x[(size_t)(t - (taps - 1) + j) * ld + c])
                               : st[(taps - 1) + src];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[idx] = from_float<T>(acc / (1.f + expf(-acc)));
  }
}

template <typename T>
__global__ void causal_conv_state_kernel(float* __restrict__ state, long state_stride,
                                         const T* __restrict__ x, int ld,
                                         const int* __restrict__ cu_tokens,
                                         const int* __restrict__ slots, int n_seqs, int channels,
                                         int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int keep = taps - 1;
  const size_t total = (size_t)n_seqs * channels;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int s = (int)(idx / channels), c = (int)(idx - (size_t)s * channels);
    const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
    float* st = state + (size_t)slots[s] * state_stride + (size_t)c * keep;
    // ascending j reads old entries at j + n >= j only: in place is safe
    for (int j = 0; j < keep; ++j) {
      const int src = n - keep + j;
      st[j] = src >= 0 ? to_float(x[(size_t)(t0 + src) * ld + c]) : st[j + n];
    }
  }
}

HB_EXPORT int hb_causal_conv_silu(void* out, const void* x, int ld, const float* w, float* state,
                                  long state_stride, const int* seq_of_token, const int* cu_tokens,
                                  const int* slots, int n_tokens, int n_seqs, int channels, int taps,
                                  int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0 || channels <= 0) return HB_OK;
  if (taps < 1 || ld < channels) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)n_tokens * channels;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(causal_conv_silu_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)out,
              (const TA*)x, ld, w, (const float*)state, state_stride, seq_of_token, cu_tokens, slots,
              n_tokens, channels, taps));
  if (taps > 1) {
    const size_t total2 = (size_t)n_seqs * channels;
    size_t blocks2 = (total2 + 255) / 256;
    if (blocks2 > 148 * 16) blocks2 = 148 * 16;
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(causal_conv_state_kernel<TA>, dim3((unsigned)blocks2), dim3(256), 0, stream, state,
                state_stride, (const TA*)x, ld, cu_tokens, slots, n_seqs, channels, taps));
  }
  return hb_check_launch();
}

// ---------------------------------------------------------------- the recurrence
constexpr int DR_CHUNK = 16;        // tokens staged in shared memory at a time
constexpr int DR_COLS = 64;         // columns of S (threads) a block owns

// qkv [T, qkv_ld]: q at q_off + kh * dk, k at k_off + kh * dk, v at v_off + h * dv
// (after convolution and silu).  beta_raw [T, beta_ld] at column h (before the sigmoid),
// a_raw [T, a_ld] at column h * dk (before dt_bias and softplus).  S of a slot at
// state + slot * state_stride, [heads, dk, dv].  o [T, heads * dv] float32.
template <typename T, int DK>
__global__ void __launch_bounds__(DR_COLS)
delta_rule_kernel(float* __restrict__ o, const T* __restrict__ qkv, int qkv_ld, int q_off, int k_off,
                  int v_off, const T* __restrict__ beta_raw, int beta_ld,
                  const T* __restrict__ a_raw, int a_ld, const float* __restrict__ a_log,
                  const float* __restrict__ dt_bias, float* __restrict__ state, long state_stride,
                  const int* __restrict__ cu_tokens, const int* __restrict__ slots, int heads,
                  int kv_heads, int dk, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* ks = sm;                              // [CHUNK][dk]
  float* qs = ks + DR_CHUNK * dk;              // [CHUNK][dk]
  float* gs = qs + DR_CHUNK * dk;              // [CHUNK][dk]
  float* vs = gs + DR_CHUNK * dk;              // [CHUNK][DR_COLS]
  float* bs = vs + DR_CHUNK * DR_COLS;         // [CHUNK]
  const int s = blockIdx.x, h = blockIdx.y;
  const int kh = h / (heads / kv_heads);
  const int col = blockIdx.z * DR_COLS + threadIdx.x;
  const bool live = col < dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
  float* S_g = state + (size_t)slots[s] * state_stride + (size_t)h * dk * dv;
  const float decay_rate = expf(a_log[h]);
  const float q_scale = rsqrtf((float)dk);

  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (live && i < dk) ? S_g[(size_t)i * dv + col] : 0.f;

  for (int c0 = 0; c0 < n; c0 += DR_CHUNK) {
    const int nc = min(DR_CHUNK, n - c0);
    __syncthreads();
    // stage the chunk: unit-norm k and q, decays, values, write strengths
    for (int j = warp; j < nc; j += DR_COLS / 32) {
      const size_t t = (size_t)(t0 + c0 + j);
      const T* kr = qkv + t * qkv_ld + k_off + (size_t)kh * dk;
      const T* qr = qkv + t * qkv_ld + q_off + (size_t)kh * dk;
      float kk = 0.f, qq = 0.f;
      for (int i = lane; i < dk; i += 32) {
        const float kv = to_float(kr[i]), qv = to_float(qr[i]);
        kk += kv * kv;
        qq += qv * qv;
      }
      const float kn = rsqrtf(warp_sum(kk) + 1e-6f), qn = rsqrtf(warp_sum(qq) + 1e-6f) * q_scale;
      for (int i = lane; i < dk; i += 32) {
        ks[j * dk + i] = to_float(kr[i]) * kn;
        qs[j * dk + i] = to_float(qr[i]) * qn;
        const float a = to_float(a_raw[t * a_ld + (size_t)h * dk + i]) + dt_bias[(size_t)h * dk + i];
        const float sp = a > 20.f ? a : log1pf(expf(a));
        gs[j * dk + i] = expf(-decay_rate * sp);
      }
      if (lane == 0) bs[j] = 1.f / (1.f + expf(-to_float(beta_raw[t * beta_ld + h])));
    }
    for (int idx = threadIdx.x; idx < nc * DR_COLS; idx += DR_COLS) {
      const int j = idx / DR_COLS, cc = idx - j * DR_COLS;
      const int vc = blockIdx.z * DR_COLS + cc;
      vs[idx] = vc < dv ? to_float(qkv[(size_t)(t0 + c0 + j) * qkv_ld + v_off + (size_t)h * dv + vc]) : 0.f;
    }
    __syncthreads();
    for (int j = 0; j < nc; ++j) {
      const float* kj = ks + j * dk;
      const float* qj = qs + j * dk;
      const float* gj = gs + j * dk;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i)
        if (i < dk) {
          S[i] *= gj[i];
          dot = fmaf(S[i], kj[i], dot);
        }
      const float u = bs[j] * (vs[j * DR_COLS + threadIdx.x] - dot);
      float out = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i)
        if (i < dk) {
          S[i] = fmaf(kj[i], u, S[i]);
          out = fmaf(S[i], qj[i], out);
        }
      if (live) o[(size_t)(t0 + c0 + j) * heads * dv + (size_t)h * dv + col] = out;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dk) S_g[(size_t)i * dv + col] = S[i];
  }
}

HB_EXPORT int hb_delta_rule(float* o, const void* qkv, int qkv_ld, int q_off, int k_off, int v_off,
                            const void* beta_raw, int beta_ld, const void* a_raw, int a_ld,
                            const float* a_log, const float* dt_bias, float* state,
                            long state_stride, const int* cu_tokens, const int* slots, int n_seqs,
                            int heads, int kv_heads, int dk, int dv, int act_dt,
                            cudaStream_t stream) {
  if (n_seqs <= 0) return HB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dk <= 0 || dk > 256 || dv <= 0 ||
      heads > 65535)
    return HB_BAD_ARGUMENT;
  dim3 grid(n_seqs, heads, (dv + DR_COLS - 1) / DR_COLS);
  const size_t smem = ((size_t)DR_CHUNK * (3 * dk + DR_COLS) + DR_CHUNK) * sizeof(float);
#define HB_DR_LAUNCH(DKMAX)                                                                       \
  HB_DISPATCH_DTYPE(act_dt, TA,                                                                   \
    if (smem > 48 * 1024)                                                                         \
      cudaFuncSetAttribute(delta_rule_kernel<TA, DKMAX>,                                          \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
    hb_launch(delta_rule_kernel<TA, DKMAX>, grid, dim3(DR_COLS), smem, stream, o, (const TA*)qkv, \
              qkv_ld, q_off, k_off, v_off, (const TA*)beta_raw, beta_ld, (const TA*)a_raw, a_ld,  \
              a_log, dt_bias, state, state_stride, cu_tokens, slots, heads, kv_heads, dk, dv))
  if (dk <= 32) HB_DR_LAUNCH(32);
  else if (dk <= 64) HB_DR_LAUNCH(64);
  else if (dk <= 128) HB_DR_LAUNCH(128);
  else HB_DR_LAUNCH(256);
#undef HB_DR_LAUNCH
  return hb_check_launch();
}

// ---------------------------------------------------------------- output norm and gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * sigmoid(gate[t, h, :]);
// one warp per (token, head); the weight (dv values) is shared by the heads.
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ o,
                                     const T* __restrict__ gate, int gate_ld,
                                     const float* __restrict__ weight, int n_rows, int heads, int dv,
                                     float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int t = row / heads, h = row - t * heads;
  const float* orow = o + (size_t)row * dv;
  const T* grow = gate + (size_t)t * gate_ld + (size_t)h * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss += orow[d] * orow[d];
  const float rstd = rsqrtf(warp_sum(ss) / (float)dv + eps);
  T* dst = out + (size_t)row * dv;
  for (int d = lane; d < dv; d += 32) {
    const float gt = 1.f / (1.f + expf(-to_float(grow[d])));
    dst[d] = from_float<T>(orow[d] * rstd * weight[d] * gt);
  }
}

HB_EXPORT int hb_gated_rmsnorm(void* out, const float* o, const void* gate, int gate_ld,
                               const float* weight, int T, int heads, int dv, float eps, int act_dt,
                               cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || dv <= 0 || gate_ld < heads * dv) return HB_BAD_ARGUMENT;
  const int n_rows = T * heads;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(gated_rmsnorm_kernel<TA>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, (TA*)out, o,
              (const TA*)gate, gate_ld, weight, n_rows, heads, dv, eps));
  return hb_check_launch();
}
