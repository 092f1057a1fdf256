// Row-wise kernels for decoders whose layers read one row of the residual stream through
// two norms at once, add a position vector to the embedding, or norm queries and keys
// per head:
//
//   embedding + sinusoid    out[t] = table[id[t]] * scale + pos(p[t]); entry 2i of pos is
//                           sin(p * f[i]), entry 2i+1 cos(p * f[i])
//   sum + RMS norm          x[r] += d0[r] + d1[r] + d2[r] + vec, then up to two normed views
//                           of the same row, out_j = x * inv * gain_j (or gathered rows
//                           without writing the stream back); one more term may be a
//                           mixture of experts' output that was never written (expert
//                           rows, their places and weights, the shared expert's part)
//   q/k norm + cache write  per head RMS norm of q and k with a gain shared by the heads,
//                           q times a temperature of the position, normed k into the key
//                           pages and k as projected into the value pages
//
// All arithmetic is fp32 with the accurate library functions; the residual stream is fp32.
#include "common.cuh"
#include "elementwise_vec.cuh"

__device__ __forceinline__ float load_any(const void* p, int code, size_t i) {
  return code == IX_F32 ? reinterpret_cast<const float*>(p)[i]
                        : __bfloat162float(reinterpret_cast<const bf16*>(p)[i]);
}

// ---------------------------------------------------------------------------
template <typename TT>
__global__ void embed_sinusoid_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                      const int* __restrict__ positions,
                                      const float* __restrict__ freq, float* __restrict__ out,
                                      int W, float scale) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const TT* row = table + (size_t)ids[t] * W;
  const float p = (float)positions[t];
  float* o = out + (size_t)t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float a = p * freq[i >> 1];
    const float pe = (i & 1) ? cosf(a) : sinf(a);
    o[i] = to_f32(row[i]) * scale + pe;
  }
}

IX_API int ix_embed_sinusoid(const void* table, int table_dtype, const int* ids,
                             const int* positions, const float* freq, int T, int W, int V,
                             float* out, float scale, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (W <= 0 || V <= 0) return IX_ERR_SIZE;
  const int threads = W >= 1024 ? 256 : 128;
  IX_DISPATCH_DTYPE(table_dtype, TT,
                    ix_launch(embed_sinusoid_kernel<TT>, dim3(T), dim3(threads), 0, stream,
                              (const TT*)table, ids, positions, freq, out, W, scale));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// sum + RMS norm.  One block per output row; the row is kept in shared memory between
// the pass that sums and the pass that scales.
// ---------------------------------------------------------------------------
template <typename TA>
__global__ void add_rmsnorm_sum_kernel(float* __restrict__ resid, const void* __restrict__ d0,
                                       int c0, const void* __restrict__ d1, int c1,
                                       const void* __restrict__ d2, int c2,
                                       const float* __restrict__ vec,
                                       const int* __restrict__ rows,
                                       const float* __restrict__ g0,
                                       const float* __restrict__ g1, TA* __restrict__ out0,
                                       TA* __restrict__ out1, int W, float eps, int write_back,
                                       const TA* __restrict__ cy, const int* __restrict__ cdest,
                                       const float* __restrict__ cw,
                                       const TA* __restrict__ cshared,
                                       const float* __restrict__ cshared_logit, int ck) {
  extern __shared__ float row[];
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const int tok = rows ? rows[r] : r;
  const size_t src = (size_t)tok * W;
  float sg = 1.0f;
  if (cshared && cshared_logit) sg = 1.0f / (1.0f + expf(-cshared_logit[tok]));
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float add = 0.f;
    bool any = false;
    if (cy) {     // a mixture's output that was never written: expert rows, weights, shared part
      for (int e = 0; e < ck; ++e)
        add += cw[(size_t)tok * ck + e] * to_f32(cy[(size_t)cdest[(size_t)tok * ck + e] * W + i]);
      if (cshared) add += sg * to_f32(cshared[src + i]);
      any = true;
    }
    if (d0) { add = any ? add + load_any(d0, c0, src + i) : load_any(d0, c0, src + i); any = true; }
    if (d1) { add = any ? add + load_any(d1, c1, src + i) : load_any(d1, c1, src + i); any = true; }
    if (d2) { add = any ? add + load_any(d2, c2, src + i) : load_any(d2, c2, src + i); any = true; }
    if (vec) { add = any ? add + vec[i] : vec[i]; any = true; }
    float v = resid[src + i];
    if (any) {
      v += add;
      if (write_back) resid[src + i] = v;
    }
    row[i] = v;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  const size_t dst = (size_t)r * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float n = row[i] * inv;
    out0[dst + i] = from_f32<TA>(n * g0[i]);
    if (out1) out1[dst + i] = from_f32<TA>(n * g1[i]);
  }
}

// Eight values of a row as fp32 from a tensor of either element type.
__device__ __forceinline__ void load8_any(const void* p, int code, size_t chunk, float* f) {
  if (code == IX_F32) {
    const float4 a = reinterpret_cast<const float4*>(p)[2 * chunk];
    const float4 b = reinterpret_cast<const float4*>(p)[2 * chunk + 1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    bf8_to_f32(reinterpret_cast<const uint4*>(p)[chunk], f);
  }
}

// bf16 outputs, width a multiple of 8 and at most 8 * NI * blockDim: the row stays in
// registers between the two passes, every access is 16 bytes.  Same sums, same order of
// the terms as the kernel above.
template <int NI>
__global__ void add_rmsnorm_sum_bf16_vec_kernel(
    float* __restrict__ resid, const void* __restrict__ d0, int c0, const void* __restrict__ d1,
    int c1, const void* __restrict__ d2, int c2, const float* __restrict__ vec,
    const int* __restrict__ rows, const float* __restrict__ g0, const float* __restrict__ g1,
    bf16* __restrict__ out0, bf16* __restrict__ out1, int W, float eps, int write_back,
    const bf16* __restrict__ cy, const int* __restrict__ cdest, const float* __restrict__ cw,
    const bf16* __restrict__ cshared, const float* __restrict__ cshared_logit, int ck) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int r = blockIdx.x;
  const int tok = rows ? rows[r] : r;
  const int chunks = W >> 3;
  const size_t src = (size_t)tok * chunks;     // in chunks of eight
  float sg = 1.0f;
  if (cshared && cshared_logit) sg = 1.0f / (1.0f + expf(-cshared_logit[tok]));
  float v[NI][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      float add[8], f[8];
      bool any = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) add[j] = 0.f;
      if (cy) {
        for (int e = 0; e < ck; ++e) {
          const float ws = cw[(size_t)tok * ck + e];
          bf8_to_f32(reinterpret_cast<const uint4*>(cy)[(size_t)cdest[(size_t)tok * ck + e] * chunks + c], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) add[j] += ws * f[j];
        }
        if (cshared) {
          bf8_to_f32(reinterpret_cast<const uint4*>(cshared)[src + c], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) add[j] += sg * f[j];
        }
        any = true;
      }
#define IX_ADD_TERM(PTR, CODE)                                  \
  if (PTR) {                                                    \
    load8_any(PTR, CODE, src + c, f);                           \
    _Pragma("unroll") for (int j = 0; j < 8; ++j) add[j] = any ? add[j] + f[j] : f[j]; \
    any = true;                                                 \
  }
      IX_ADD_TERM(d0, c0)
      IX_ADD_TERM(d1, c1)
      IX_ADD_TERM(d2, c2)
#undef IX_ADD_TERM
      if (vec) {
        load8_any(vec, IX_F32, c, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) add[j] = any ? add[j] + f[j] : f[j];
        any = true;
      }
      load8_any(resid, IX_F32, src + c, v[i]);
      if (any) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] += add[j];
        if (write_back) {
          float4* x = reinterpret_cast<float4*>(resid) + 2 * (src + c);
          x[0] = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
          x[1] = make_float4(v[i][4], v[i][5], v[i][6], v[i][7]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
  const size_t dst = (size_t)r * chunks;
#pragma unroll
  for (int i = 0; i < NI; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < chunks) {
      float g[8], f[8];
      load8_any(g0, IX_F32, c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = v[i][j] * inv * g[j];
      reinterpret_cast<uint4*>(out0)[dst + c] = f32_to_bf8(f);
      if (out1) {
        load8_any(g1, IX_F32, c, g);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = v[i][j] * inv * g[j];
        reinterpret_cast<uint4*>(out1)[dst + c] = f32_to_bf8(f);
      }
    }
  }
}

IX_API int ix_add_rmsnorm_sum(float* resid, const void* d0, int c0, const void* d1, int c1,
                              const void* d2, int c2, const float* vec, const int* rows,
                              const float* g0, const float* g1, void* out0, void* out1,
                              int out_dtype, int R, int W, float eps, int write_back,
                              const void* cy, const int* cdest, const float* cw,
                              const void* cshared, const float* cshared_logit, int ck,
                              cudaStream_t stream) {
  if (R <= 0) return IX_OK;
  if (W <= 0 || !g0 || !out0 || (out1 && !g1)) return IX_ERR_SIZE;
  if (cy && (!cdest || !cw || ck <= 0)) return IX_ERR_SIZE;
  const uintptr_t all = (uintptr_t)resid | (uintptr_t)d0 | (uintptr_t)d1 | (uintptr_t)d2 |
                        (uintptr_t)vec | (uintptr_t)g0 | (uintptr_t)g1 | (uintptr_t)out0 |
                        (uintptr_t)out1 | (uintptr_t)cy | (uintptr_t)cshared;
  if (out_dtype == IX_BF16 && W % 8 == 0 && (all & 15) == 0 && W <= 8 * 4 * 256) {
    const int chunks = W / 8;
    const int vt = chunks >= 256 ? 256 : (chunks >= 128 ? 128 : 64);
    const int ni = (chunks + vt - 1) / vt;
#define IX_ARS(NI)                                                                            \
  ix_launch(add_rmsnorm_sum_bf16_vec_kernel<NI>, dim3(R), dim3(vt), 0, stream, resid, d0, c0, \
            d1, c1, d2, c2, vec, rows, g0, g1, (bf16*)out0, (bf16*)out1, W, eps, write_back,  \
            (const bf16*)cy, cdest, cw, (const bf16*)cshared, cshared_logit, ck)
    if (ni == 1) IX_ARS(1);
    else if (ni == 2) IX_ARS(2);
    else IX_ARS(4);
#undef IX_ARS
    return ix_launch_status();
  }
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  IX_DISPATCH_DTYPE(out_dtype, TA, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(add_rmsnorm_sum_kernel<TA>,
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ix_launch(add_rmsnorm_sum_kernel<TA>, dim3(R), dim3(threads), smem, stream, resid, d0, c0, d1,
              c1, d2, c2, vec, rows, g0, g1, (TA*)out0, (TA*)out1, W, eps, write_back,
              (const TA*)cy, cdest, cw, (const TA*)cshared, cshared_logit, ck);
  });
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// q/k norm + cache write.  One warp per (token, head); heads 0..H-1 are queries, the
// following G are key/value heads.  qk row layout: [H * D | G * D].
// ---------------------------------------------------------------------------

#define QKN_WARPS 4

template <typename TA>
__global__ void qk_norm_append_kernel(const TA* __restrict__ qk, const float* __restrict__ q_gain,
                                      const float* __restrict__ k_gain,
                                      const int* __restrict__ positions, TA* __restrict__ q_out,
                                      TA* __restrict__ k_cache, TA* __restrict__ v_cache,
                                      const int* __restrict__ slots, int H, int G, int D,
                                      int page_size, float eps, float temp_coef, int temp_every) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int j = blockIdx.y * QKN_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (j >= H + G) return;
  const TA* src = qk + (size_t)t * (H + G) * D + (size_t)j * D;
  float ss = 0.f;
  for (int d = lane; d < D; d += 32) {
    const float v = to_f32(src[d]);
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
  if (j < H) {
    float temp = 1.0f;
    if (temp_every > 0)
      temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);
    TA* dst = q_out + ((size_t)t * H + j) * D;
    for (int d = lane; d < D; d += 32)
      dst[d] = from_f32<TA>(to_f32(src[d]) * inv * q_gain[d] * temp);
  } else if (k_cache) {
    const int g = j - H;
    const int slot = slots[t];
    if (slot < 0) return;
    const size_t base = (((size_t)(slot / page_size) * G + g) * page_size + slot % page_size) * D;
    for (int d = lane; d < D; d += 32) {
      v_cache[base + d] = src[d];
      k_cache[base + d] = from_f32<TA>(to_f32(src[d]) * inv * k_gain[d]);
    }
  }
}

// bf16, D a multiple of 8 with D / 8 a power of two up to 32: GL = D / 8 lanes share a
// head, each with eight values in one 16-byte access, 32 / GL heads a warp.
template <int GL>
__global__ void qk_norm_append_bf16_vec_kernel(
    const bf16* __restrict__ qk, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, const int* __restrict__ positions, bf16* __restrict__ q_out,
    bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, const int* __restrict__ slots, int H,
    int G, int D, int page_size, float eps, float temp_coef, int temp_every) {
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31;
  constexpr int HPW = 32 / GL;
  const int j = (blockIdx.y * QKN_WARPS + (threadIdx.x >> 5)) * HPW + lane / GL;
  const int sub = lane % GL;
  const bool ok = j < H + G;
  float f[8];
  uint4 raw = make_uint4(0u, 0u, 0u, 0u);
  if (ok) raw = reinterpret_cast<const uint4*>(qk + (size_t)t * (H + G) * D + (size_t)j * D)[sub];
  bf8_to_f32(raw, f);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
#pragma unroll
  for (int d = GL / 2; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  if (!ok) return;
  const float inv = 1.0f / sqrtf(ss / (float)D + eps);
  float g[8];
  if (j < H) {
    float temp = 1.0f;
    if (temp_every > 0)
      temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);
    load8_any(q_gain, IX_F32, sub, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i] * temp;
    reinterpret_cast<uint4*>(q_out + ((size_t)t * H + j) * D)[sub] = f32_to_bf8(f);
  } else if (k_cache) {
    const int slot = slots[t];
    if (slot < 0) return;
    const size_t base =
        (((size_t)(slot / page_size) * G + (j - H)) * page_size + slot % page_size) * D;
    reinterpret_cast<uint4*>(v_cache + base)[sub] = raw;
    load8_any(k_gain, IX_F32, sub, g);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = f[i] * inv * g[i];
    reinterpret_cast<uint4*>(k_cache + base)[sub] = f32_to_bf8(f);
  }
}

IX_API int ix_qk_norm_append(const void* qk, int dtype, const float* q_gain, const float* k_gain,
                             const int* positions, void* q_out, void* k_cache, void* v_cache,
                             const int* slots, int T, int H, int G, int D, int page_size,
                             float eps, float temp_coef, int temp_every, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || G <= 0 || D <= 0 || page_size <= 0 || temp_every < 0) return IX_ERR_SIZE;
  if ((k_cache != nullptr) != (v_cache != nullptr) || (k_cache && !slots)) return IX_ERR_SIZE;
  const int groups = (H + G + QKN_WARPS - 1) / QKN_WARPS;
  if (groups > 65535) return IX_ERR_SIZE;
  const int gl = D / 8;
  if (dtype == IX_BF16 && D % 8 == 0 && gl <= 32 && (gl & (gl - 1)) == 0 &&
      (((uintptr_t)qk | (uintptr_t)q_gain | (uintptr_t)k_gain | (uintptr_t)q_out |
        (uintptr_t)k_cache | (uintptr_t)v_cache) & 15) == 0) {
    const int hpb = QKN_WARPS * (32 / gl);
    const int vgroups = (H + G + hpb - 1) / hpb;
#define IX_QKN(GL)                                                                              \
  ix_launch(qk_norm_append_bf16_vec_kernel<GL>, dim3(T, vgroups), dim3(32 * QKN_WARPS), 0,      \
            stream, (const bf16*)qk, q_gain, k_gain, positions, (bf16*)q_out, (bf16*)k_cache,   \
            (bf16*)v_cache, slots, H, G, D, page_size, eps, temp_coef, temp_every)
    if (gl == 32) IX_QKN(32);
    else if (gl == 16) IX_QKN(16);
    else if (gl == 8) IX_QKN(8);
    else if (gl == 4) IX_QKN(4);
    else if (gl == 2) IX_QKN(2);
    else IX_QKN(1);
#undef IX_QKN
    return ix_launch_status();
  }
  IX_DISPATCH_DTYPE(dtype, TA,
                    ix_launch(qk_norm_append_kernel<TA>, dim3(T, groups), dim3(32 * QKN_WARPS), 0,
                              stream, (const TA*)qk, q_gain, k_gain, positions, (TA*)q_out,
                              (TA*)k_cache, (TA*)v_cache, slots, H, G, D, page_size, eps,
                              temp_coef, temp_every));
  return ix_launch_status();
}
