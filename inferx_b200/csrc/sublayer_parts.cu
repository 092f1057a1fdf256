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
#include "elementwise_vec.cuh"

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

// bf16 output, width a multiple of 8: eight values a thread, 16-byte accesses
__global__ void token_shift_bf16_vec_kernel(const float* __restrict__ resid,
                                            const float* __restrict__ mix, float* __restrict__ state,
                                            const int* __restrict__ cu_q,
                                            const int* __restrict__ seq_of_token,
                                            const int* __restrict__ state_slot,
                                            bf16* __restrict__ out, int W) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int s = seq_of_token[t];
  const bool first = (t == cu_q[s]);
  const float4* x = reinterpret_cast<const float4*>(resid + (size_t)t * W);
  float4* st = reinterpret_cast<float4*>(state + (size_t)state_slot[s] * W);
  const float4* prev = first ? st : x - W / 4;
  const float4* last = reinterpret_cast<const float4*>(resid + (size_t)(cu_q[s + 1] - 1) * W);
  const float4* mx = reinterpret_cast<const float4*>(mix);
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * W);
  for (int c = threadIdx.x; c < W / 8; c += blockDim.x) {
    const float4 a0 = x[2 * c], a1 = x[2 * c + 1], p0 = prev[2 * c], p1 = prev[2 * c + 1];
    const float4 m0 = mx[2 * c], m1 = mx[2 * c + 1];
    float f[8] = {a0.x + (p0.x - a0.x) * m0.x, a0.y + (p0.y - a0.y) * m0.y,
                  a0.z + (p0.z - a0.z) * m0.z, a0.w + (p0.w - a0.w) * m0.w,
                  a1.x + (p1.x - a1.x) * m1.x, a1.y + (p1.y - a1.y) * m1.y,
                  a1.z + (p1.z - a1.z) * m1.z, a1.w + (p1.w - a1.w) * m1.w};
    o[c] = f32_to_bf8(f);
    if (first) {
      st[2 * c] = last[2 * c];
      st[2 * c + 1] = last[2 * c + 1];
    }
  }
}

IX_API int ix_token_shift(const float* resid, const float* mix, float* state, const int* cu_q,
                          const int* seq_of_token, const int* state_slot, void* out,
                          int out_dtype, int T, int W, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0) return IX_ERR_SIZE;
  const int threads = W >= 1024 ? 256 : 128;
  if (out_dtype == IX_BF16 && W % 8 == 0 &&
      (((uintptr_t)resid | (uintptr_t)mix | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
    ix_launch(token_shift_bf16_vec_kernel, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream, resid,
              mix, state, cu_q, seq_of_token, state_slot, (bf16*)out, W);
    return ix_launch_status();
  }
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

// Parts that are a multiple of 8 entries with a bf16 copy of the result: eight values a
// thread and pass, 16-byte accesses.  The sum of squares is formed in the same order
// whatever the batch (it depends on the part's size and the block's only).
template <typename TD> struct Load8;
template <> struct Load8<float> {
  static __device__ __forceinline__ void at(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};
template <> struct Load8<bf16> {
  static __device__ __forceinline__ void at(const bf16* p, float* f) {
    bf8_to_f32(*reinterpret_cast<const uint4*>(p), f);
  }
};

template <typename TD, bool CAST>
__global__ void group_norm_add_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                          const float* __restrict__ gain, bf16* __restrict__ cast,
                                          int W, int part, float eps) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const size_t base = (size_t)blockIdx.x * W + (size_t)blockIdx.y * part;
  const TD* d = delta + base;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part / 8; c += blockDim.x) {
    float f[8];
    Load8<TD>::at(d + 8 * c, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
  const float* g = gain + (size_t)blockIdx.y * part;
  float* x = resid + base;
  for (int c = threadIdx.x; c < part / 8; c += blockDim.x) {
    float f[8], r[8], w[8];
    Load8<TD>::at(d + 8 * c, f);
    Load8<float>::at(x + 8 * c, r);
    Load8<float>::at(g + 8 * c, w);
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] += f[j] * inv * w[j];
    *reinterpret_cast<float4*>(x + 8 * c) = make_float4(r[0], r[1], r[2], r[3]);
    *reinterpret_cast<float4*>(x + 8 * c + 4) = make_float4(r[4], r[5], r[6], r[7]);
    if (CAST) *reinterpret_cast<uint4*>(cast + base + 8 * c) = f32_to_bf8(r);
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
  if (part % 8 == 0 && (cast == nullptr || cast_dtype == IX_BF16) &&
      (((uintptr_t)resid | (uintptr_t)delta | (uintptr_t)gain | (uintptr_t)cast) & 15) == 0) {
    int th = 32;
    while (th < 256 && th * 8 < part) th *= 2;
    const dim3 vgrid(T, groups), vblock(th);
#define IX_GNV(TD, CAST)                                                                       \
  ix_launch(group_norm_add_vec_kernel<TD, CAST>, vgrid, vblock, 0, stream, resid,                \
            (const TD*)delta, gain, (bf16*)cast, W, part, eps)
    if (delta_dtype == IX_F32) {
      if (cast) IX_GNV(float, true); else IX_GNV(float, false);
    } else if (delta_dtype == IX_BF16) {
      if (cast) IX_GNV(bf16, true); else IX_GNV(bf16, false);
    } else {
      return IX_ERR_DTYPE;
    }
#undef IX_GNV
    return ix_launch_status();
  }
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

// bf16 rows of 8-element chunks, fast exponential and reciprocal (their error is far below a
// bf16 ulp), two chunks a pass
__global__ void __launch_bounds__(256)
glu_clamped_bf16_vec_kernel(const uint4* __restrict__ gu, uint4* __restrict__ out,
                            unsigned total_chunks, unsigned chunks_per_row, float limit,
                            float alpha, float up_shift) {
  IX_PDL_WAIT();
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < total_chunks; i0 += 2 * stride) {
    const unsigned i1 = i0 + stride;
    const bool two = i1 < total_chunks;
    const unsigned t0 = i0 / chunks_per_row, t1 = two ? i1 / chunks_per_row : t0;
    const size_t a0 = (size_t)t0 * chunks_per_row + i0;          // t * 2 * cpr + c
    const size_t a1 = two ? (size_t)t1 * chunks_per_row + i1 : a0;
    const uint4 g0 = gu[a0], u0 = gu[a0 + chunks_per_row];
    const uint4 g1 = gu[a1], u1 = gu[a1 + chunks_per_row];
    float g[8], u[8], o[8];
    bf8_to_f32(g0, g);
    bf8_to_f32(u0, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gg = fminf(g[j], limit), uu = fminf(fmaxf(u[j], -limit), limit);
      o[j] = __fdividef(gg, 1.0f + __expf(-alpha * gg)) * (uu + up_shift);
    }
    out[i0] = f32_to_bf8(o);
    if (two) {
      bf8_to_f32(g1, g);
      bf8_to_f32(u1, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gg = fminf(g[j], limit), uu = fminf(fmaxf(u[j], -limit), limit);
        o[j] = __fdividef(gg, 1.0f + __expf(-alpha * gg)) * (uu + up_shift);
      }
      out[i1] = f32_to_bf8(o);
    }
  }
}

IX_API int ix_glu_clamped(const void* gu, void* out, int act_dtype, int T, int I, float limit,
                          float alpha, float up_shift, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (I <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * I;
  if (act_dtype == IX_BF16 && I % 8 == 0 && (((uintptr_t)gu | (uintptr_t)out) & 15) == 0 &&
      total / 8 < (1LL << 30)) {
    const long long chunks = total / 8;
    long long vb = (chunks + 511) / 512;
    if (vb > 148 * 8) vb = 148 * 8;
    ix_launch(glu_clamped_bf16_vec_kernel, dim3((int)vb), dim3(256), 0, stream, (const uint4*)gu,
              (uint4*)out, (unsigned)chunks, (unsigned)(I / 8), limit, alpha, up_shift);
    return ix_launch_status();
  }
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

// bf16, D and the gate's row length multiples of 8: one 16-byte chunk a thread and pass
__global__ void gate_heads_bf16_vec_kernel(const uint4* __restrict__ o, const bf16* __restrict__ gate,
                                           long long gate_ld, uint4* __restrict__ out, int T, int H,
                                           int D8) {
  IX_PDL_WAIT();
  const long long total = (long long)T * H * D8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / ((long long)H * D8);
    const int c = (int)(idx - t * H * D8);
    const int h = c / D8, j = c - h * D8;
    float v[8], g[8];
    bf8_to_f32(o[((size_t)h * T + t) * D8 + j], v);
    bf8_to_f32(*reinterpret_cast<const uint4*>(gate + t * gate_ld + (size_t)c * 8), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = __fdividef(v[k], 1.0f + __expf(-g[k]));
    out[idx] = f32_to_bf8(v);
  }
}

IX_API int ix_gate_heads(const void* o, const void* gate, long long gate_ld, void* out,
                         int act_dtype, int T, int H, int D, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || D <= 0) return IX_ERR_SIZE;
  const long long total = (long long)T * H * D;
  if (act_dtype == IX_BF16 && D % 8 == 0 && gate_ld % 8 == 0 &&
      (((uintptr_t)o | (uintptr_t)gate | (uintptr_t)out) & 15) == 0) {
    long long vb = (total / 8 + 255) / 256;
    if (vb > 148 * 16) vb = 148 * 16;
    ix_launch(gate_heads_bf16_vec_kernel, dim3((int)vb), dim3(256), 0, stream, (const uint4*)o,
              (const bf16*)gate, gate_ld, (uint4*)out, T, H, D / 8);
    return ix_launch_status();
  }
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    ix_launch(gate_heads_kernel<TA>, dim3((int)blocks), dim3(256), 0, stream,
                              (const TA*)o, (const TA*)gate, gate_ld, (TA*)out, T, H, D));
  return ix_launch_status();
}
