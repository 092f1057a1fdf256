// Row-wise kernels for decoders that normalise a sublayer's OUTPUT before adding it
// to the residual stream, mix each token's input with the previous token's, and gate
// or clamp inside their sublayers:
//
//   token shift           out[t] = x[t] + (x[t-1] - x[t]) * mix, the row before a
//                         sequence's first token taken from per-request state, which
//                         is then replaced by the sequence's last row
//   grouped RMS norm      a row in G equal consecutive parts, each over its own root
//                         mean square; either added into the residual stream
//                         (resid += norm(delta) * gain) or gathered for the head
//   clamped GLU           min(g, L) * sigmoid(a * min(g, L)) * (clamp(u, -L, L) + b)
//   sigmoid output gate   out[t, h, :] = o[h, t, :] * sigmoid(gate[t, h, :])
//
// All arithmetic is fp32; the residual stream and the state are fp32 tensors.
#include "common.cuh"

// ---------------------------------------------------------------------------
// token shift.  One block per token.  The block of a sequence's first token reads
// the state row and afterwards stores the sequence's last row of this step there;
// each thread touches the same elements in both, so the read precedes the write.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void token_shift_kernel(const float* __restrict__ resid, const float* __restrict__ mix,
                                   float* __restrict__ state, const int* __restrict__ cu_q,
                                   const int* __restrict__ seq_of_token,
                                   const int* __restrict__ state_slot, TA* __restrict__ out, int W) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const bool first = (t == cu_q[s]);
  const float* x = resid + (size_t)t * W;
  float* st = state + (size_t)state_slot[s] * W;
  const float* prev = first ? st : x - W;
  TA* o = out + (size_t)t * W;
  const float* last = resid + (size_t)(cu_q[s + 1] - 1) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = x[i];
    const float p = prev[i];
    o[i] = from_f32<TA>(v + (p - v) * mix[i]);
    if (first) st[i] = last[i];
  }
}

IX_API int ix_token_shift(const float* resid, const float* mix, float* state, const int* cu_q,
                          const int* seq_of_token, const int* state_slot, void* out,
                          int out_dtype, int T, int W, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0) return IX_ERR_SIZE;
  const int threads = W >= 1024 ? 256 : 128;
  IX_DISPATCH_DTYPE(out_dtype, TA,
                    ix_launch(token_shift_kernel<TA>, dim3(T), dim3(threads), 0, stream, resid, mix,
                              state, cu_q, seq_of_token, state_slot, (TA*)out, W));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// grouped RMS norm.  One block per (row, group).
//   add form:   v = delta[r, part];  resid[r, part] += v * inv * gain;  cast[r, part] = resid
//   rows form:  v = resid[rows[r], part];  out[r, part] = v * inv * gain
// inv = 1 / sqrt(mean(v^2) + eps) over the part.
// ---------------------------------------------------------------------------
template <typename TD, typename TA>
__global__ void group_norm_add_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                      const float* __restrict__ gain, TA* __restrict__ cast,
                                      int W, int part, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const size_t base = (size_t)blockIdx.x * W + (size_t)blockIdx.y * part;
  const TD* d = delta + base;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = to_f32(d[i]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
  const float* g = gain + (size_t)blockIdx.y * part;
  float* x = resid + base;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float v = x[i] + to_f32(d[i]) * inv * g[i];
    x[i] = v;
    if (cast) cast[base + i] = from_f32<TA>(v);
  }
}

template <typename TA>
__global__ void group_norm_rows_kernel(const float* __restrict__ resid, const int* __restrict__ rows,
                                       const float* __restrict__ gain, TA* __restrict__ out, int W,
                                       int part, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const size_t src = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  const float* x = resid + src * W + (size_t)blockIdx.y * part;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) ss += x[i] * x[i];
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
  const float* g = gain + (size_t)blockIdx.y * part;
  TA* o = out + (size_t)blockIdx.x * W + (size_t)blockIdx.y * part;
  for (int i = threadIdx.x; i < part; i += blockDim.x) o[i] = from_f32<TA>(x[i] * inv * g[i]);
}

static inline int norm_threads(int part) {
  int t = 32;
  while (t < 256 && t * 4 < part) t *= 2;
  return t;
}

// delta: [T, W] of delta_dtype; cast (optional): [T, W] of cast_dtype
IX_API int ix_group_norm_add(float* resid, const void* delta, int delta_dtype, const float* gain,
                             void* cast, int cast_dtype, int T, int W, int groups, float eps,
                             cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0 || groups <= 0 || W % groups || groups > 65535) return IX_ERR_SIZE;
  const int part = W / groups;
  const dim3 grid(T, groups), block(norm_threads(part));
#define IX_GNA(TD, TA)                                                                         \
  ix_launch(group_norm_add_kernel<TD, TA>, grid, block, 0, stream, resid, (const TD*)delta, gain, \
            (TA*)cast, W, part, eps)
  if (delta_dtype == IX_F32 && cast_dtype == IX_F32) IX_GNA(float, float);
  else if (delta_dtype == IX_F32 && cast_dtype == IX_BF16) IX_GNA(float, bf16);
  else if (delta_dtype == IX_BF16 && cast_dtype == IX_BF16) IX_GNA(bf16, bf16);
  else if (delta_dtype == IX_BF16 && cast_dtype == IX_F32) IX_GNA(bf16, float);
  else return IX_ERR_DTYPE;
#undef IX_GNA
  return ix_launch_status();
}

IX_API int ix_group_norm_rows(const float* resid, const int* rows, const float* gain, void* out,
                              int out_dtype, int R, int W, int groups, float eps,
                              cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (W <= 0 || groups <= 0 || W % groups || groups > 65535) return IX_ERR_SIZE;
  const int part = W / groups;
  const dim3 grid(R, groups), block(norm_threads(part));
  IX_DISPATCH_DTYPE(out_dtype, TA,
                    ix_launch(group_norm_rows_kernel<TA>, grid, block, 0, stream, resid, rows, gain,
                              (TA*)out, W, part, eps));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// clamped GLU on a fused [T, 2I] product (gate columns, then up columns)
// ---------------------------------------------------------------------------
__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha,
                                             float up_shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-alpha * g)) * (u + up_shift);
}

template <typename TA>
__global__ void glu_clamped_kernel(const TA* __restrict__ gu, TA* __restrict__ out, long long total,
                                   int I, float limit, float alpha, float up_shift) {
  IX_PDL_WAIT();
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / I;
    const int j = (int)(idx - t * I);
    const float g = to_f32(gu[t * 2 * I + j]);
    const float u = to_f32(gu[t * 2 * I + I + j]);
    out[idx] = from_f32<TA>(clamped_glu(g, u, limit, alpha, up_shift));
  }
}

IX_API int ix_glu_clamped(const void* gu, void* out, int act_dtype, int T, int I, float limit,
                          float alpha, float up_shift, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (I <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * I;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    ix_launch(glu_clamped_kernel<TA>, dim3((int)blocks), dim3(256), 0, stream,
                              (const TA*)gu, (TA*)out, total, I, limit, alpha, up_shift));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// sigmoid output gate with the heads brought back beside each other:
//   out[t, h * D + j] = o[h, t, j] * sigmoid(gate[t * gate_ld + h * D + j])
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void gate_heads_kernel(const TA* __restrict__ o, const TA* __restrict__ gate,
                                  long long gate_ld, TA* __restrict__ out, int T, int H, int D) {
  IX_PDL_WAIT();
  const long long total = (long long)T * H * D;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / ((long long)H * D);
    const int c = (int)(idx - t * H * D);
    const int h = c / D, j = c - h * D;
    const float v = to_f32(o[((size_t)h * T + t) * D + j]);
    const float g = to_f32(gate[t * gate_ld + c]);
    out[idx] = from_f32<TA>(v / (1.0f + expf(-g)));
  }
}

IX_API int ix_gate_heads(const void* o, const void* gate, long long gate_ld, void* out,
                         int act_dtype, int T, int H, int D, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || D <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * H * D;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    ix_launch(gate_heads_kernel<TA>, dim3((int)blocks), dim3(256), 0, stream,
                              (const TA*)o, (const TA*)gate, gate_ld, (TA*)out, T, H, D));
  return ix_launch_status();
}
