// Attention over a cache of latents: every token keeps one record
//   [ c (rank values, RMS-normed) | k_rot (dr values, rotated) ]
// shared by all heads.  A head's key would be (W_uk c | k_rot) and its value W_uv c;
// with the key matrix folded into the query (q_lat = W_uk^T q_plain, done by the
// caller as a product batched over heads) the score is
//   (q_lat . c + q_rot . k_rot) * scale
// and the head's output in latent space is sum_j p_j c_j, which the caller widens
// with W_uv.  So this is one-key-head attention whose keys are the whole record and
// whose values are the record's first `rank` entries.
//
//   ix_latent_prepare    per token: RMS norm of the latent (fp32), interleaved rotation
//                        of the shared key part and of every head's rotated query
//                        part (angles, cos and sin in fp32), record written into its
//                        cache slot; the plain query parts laid out heads outermost
//                        for the product with the folded key matrix
//   ix_latent_attention  general kernel: any sizes, fp32 arithmetic, either element
//                        type; one warp per (token, head), keys in tiles of 32 that
//                        start on multiples of 32 of the absolute position, so that a
//                        row's result does not depend on how the step was batched
#include "common.cuh"

// ---------------------------------------------------------------------------
// prepare.  proj: [T, ld]; the queries of head h start at column q_off + h * (dn + dr)
// (dn plain, then dr rotated), the down-projection at kv_off (rank, then dr).
// Pair i < rot_dims / 2 of a rotated part is (2i, 2i+1), turned by pos * freq[i];
// cos and sin are multiplied by `mag`; entries from rot_dims on pass unchanged.
// ---------------------------------------------------------------------------
#define LP_HEADS 4   // heads a block of the preparation handles

template <typename TA>
__global__ void latent_prepare_kernel(const TA* __restrict__ proj, long long ld, int q_off,
                                      int kv_off, const int* __restrict__ positions,
                                      const float* __restrict__ freq, float mag,
                                      const float* __restrict__ gain, float eps,
                                      const int* __restrict__ slots, TA* __restrict__ cache,
                                      TA* __restrict__ q_rot, TA* __restrict__ q_plain, int T, int H,
                                      int dn, int dr, int rot_dims, int rank) {
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int t = blockIdx.x;
  const TA* row = proj + (size_t)t * ld;
  const float pos = (float)positions[t];
  const int half = rot_dims >> 1;
  // blockIdx.y: a group of LP_HEADS heads; the first group also makes the token's record
  const int h_lo = blockIdx.y * LP_HEADS, h_n = min(LP_HEADS, H - h_lo);
  if (cache != nullptr && blockIdx.y == 0) {
    const TA* kv = row + kv_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) {
      const float v = to_f32(kv[i]);
      ss += v * v;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)rank + eps);
    TA* rec = cache + (size_t)slots[t] * (rank + dr);
    for (int i = threadIdx.x; i < rank; i += blockDim.x)
      rec[i] = from_f32<TA>(to_f32(kv[i]) * inv * gain[i]);
    for (int p = threadIdx.x; p < (dr + 1) / 2; p += blockDim.x) {
      const float u = to_f32(kv[rank + 2 * p]);
      const float v = 2 * p + 1 < dr ? to_f32(kv[rank + 2 * p + 1]) : 0.f;
      float a = u, b = v;
      if (p < half) {
        const float ang = pos * freq[p];
        const float c = cosf(ang) * mag, s = sinf(ang) * mag;
        a = u * c - v * s;
        b = v * c + u * s;
      }
      rec[rank + 2 * p] = from_f32<TA>(a);
      if (2 * p + 1 < dr) rec[rank + 2 * p + 1] = from_f32<TA>(b);
    }
  }
  // the plain query parts, heads outermost: [H, T, dn]
  for (int idx = threadIdx.x; idx < h_n * dn; idx += blockDim.x) {
    const int h = h_lo + idx / dn, d = idx % dn;
    q_plain[((size_t)h * T + t) * dn + d] = row[q_off + (size_t)h * (dn + dr) + d];
  }
  const int pairs = (dr + 1) / 2;
  for (int idx = threadIdx.x; idx < h_n * pairs; idx += blockDim.x) {
    const int h = h_lo + idx / pairs, p = idx % pairs;
    const TA* q = row + q_off + (size_t)h * (dn + dr) + dn;
    const float u = to_f32(q[2 * p]);
    const float v = 2 * p + 1 < dr ? to_f32(q[2 * p + 1]) : 0.f;
    float a = u, b = v;
    if (p < half) {
      const float ang = pos * freq[p];
      const float c = cosf(ang) * mag, s = sinf(ang) * mag;
      a = u * c - v * s;
      b = v * c + u * s;
    }
    TA* o = q_rot + ((size_t)t * H + h) * dr;
    o[2 * p] = from_f32<TA>(a);
    if (2 * p + 1 < dr) o[2 * p + 1] = from_f32<TA>(b);
  }
}

IX_API int ix_latent_prepare(const void* proj, long long ld, int q_off, int kv_off,
                             const int* positions, const float* freq, float mag,
                             const float* gain, float eps, const int* slots, void* cache,
                             void* q_rot, void* q_plain, int act_dtype, int T, int H, int dn,
                             int dr, int rot_dims, int rank, cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || dn < 0 || dr < 0 || rank <= 0 || rot_dims < 0 || rot_dims > dr || rot_dims % 2)
    return IX_ERR_SIZE;
  if (cache != nullptr && slots == nullptr) return IX_ERR_SIZE;
  IX_DISPATCH_DTYPE(act_dtype, TA,
                    ix_launch(latent_prepare_kernel<TA>, dim3(T, (H + LP_HEADS - 1) / LP_HEADS),
                              dim3(128), 0, stream,
                              (const TA*)proj, ld, q_off, kv_off, positions, freq, mag, gain, eps,
                              slots, (TA*)cache, (TA*)q_rot, (TA*)q_plain, T, H, dn, dr, rot_dims,
                              rank));
  return ix_launch_status();
}

// ---------------------------------------------------------------------------
// general attention kernel
// ---------------------------------------------------------------------------
#define LA_KT 32   // keys per tile
#define LA_HB 8    // heads (warps) per block

template <typename TA, int NR>
__global__ void __launch_bounds__(LA_HB * 32)
latent_attention_kernel(const TA* __restrict__ q_lat, long long ql_sh, long long ql_st,
                        const TA* __restrict__ q_rot, const TA* __restrict__ cache,
                        const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                        TA* __restrict__ out, long long o_sh, long long o_st, int H, int rank,
                        int dr, int page, int window, float scale) {
  extern __shared__ float la_smem[];
  __shared__ int key_row[LA_KT];
  IX_PDL_WAIT();
  const int Dk = rank + dr;
  const int ldk = Dk + 1;
  float* qs = la_smem;                     // [LA_HB][Dk]
  float* ks = la_smem + LA_HB * Dk;        // [LA_KT][Dk + 1]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * LA_HB + warp;
  const int s = seq_of_token[t];
  const int pos = positions[t];
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (h < H) {
    const TA* ql = q_lat + (size_t)h * ql_sh + (size_t)t * ql_st;
    const TA* qr = q_rot + ((size_t)t * H + h) * dr;
    for (int d = lane; d < rank; d += 32) qs[warp * Dk + d] = to_f32(ql[d]);
    for (int d = lane; d < dr; d += 32) qs[warp * Dk + rank + d] = to_f32(qr[d]);
  }
  float m = -INFINITY, l = 0.f;
  float o[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) o[i] = 0.f;
  const int* table = block_table + (size_t)s * max_blocks;
  for (int k0 = (lo / LA_KT) * LA_KT; k0 <= pos; k0 += LA_KT) {
    __syncthreads();   // the previous tile is no longer read (and qs is written)
    if (threadIdx.x < LA_KT) {
      const int kp = k0 + threadIdx.x;
      int r = -1;
      if (kp >= lo && kp <= pos) {
        const int pg = table[kp / page];
        if (pg >= 0) r = pg * page + kp % page;
      }
      key_row[threadIdx.x] = r;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < LA_KT * Dk; idx += blockDim.x) {
      const int j = idx / Dk, d = idx - j * Dk;
      const int r = key_row[j];
      ks[j * ldk + d] = r >= 0 ? to_f32(cache[(size_t)r * Dk + d]) : 0.f;
    }
    __syncthreads();
    if (h < H) {
      const bool valid = key_row[lane] >= 0;
      float sc = 0.f;
      const float* kq = ks + lane * ldk;
      const float* qq = qs + warp * Dk;
      for (int d = 0; d < Dk; ++d) sc += qq[d] * kq[d];
      sc = valid ? sc * scale : -INFINITY;
      const float m_new = fmaxf(m, warp_max(sc));
      const float p = valid ? expf(sc - m_new) : 0.f;
      const float corr = expf(m - m_new);     // 0 at the first tile (m = -inf)
      l = l * corr + warp_sum(p);
      m = m_new;
#pragma unroll
      for (int i = 0; i < NR; ++i) o[i] *= corr;
      for (int j = 0; j < LA_KT; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const float* kv = ks + j * ldk;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
          const int d = lane + 32 * i;
          if (d < rank) o[i] += pj * kv[d];
        }
      }
    }
  }
  if (h < H) {
    const float inv = 1.0f / l;
    TA* dst = out + (size_t)h * o_sh + (size_t)t * o_st;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int d = lane + 32 * i;
      if (d < rank) dst[d] = from_f32<TA>(o[i] * inv);
    }
  }
}

IX_API int ix_latent_attention_max_rank() { return 1024; }

template <typename TA, int NR>
static int launch_latent_attention(const void* q_lat, long long ql_sh, long long ql_st,
                                   const void* q_rot, const void* cache, const int* block_table,
                                   int max_blocks, const int* seq_of_token, const int* positions,
                                   void* out, long long o_sh, long long o_st, int T, int H,
                                   int rank, int dr, int page, int window, float scale,
                                   cudaStream_t stream) {
  const int Dk = rank + dr;
  const size_t smem = ((size_t)LA_HB * Dk + (size_t)LA_KT * (Dk + 1)) * sizeof(float);
  if (smem > 200 * 1024) return IX_ERR_SMEM;
  auto kern = latent_attention_kernel<TA, NR>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  ix_launch(kern, dim3(T, (H + LA_HB - 1) / LA_HB), dim3(LA_HB * 32), smem, stream,
            (const TA*)q_lat, ql_sh, ql_st, (const TA*)q_rot, (const TA*)cache, block_table,
            max_blocks, seq_of_token, positions, (TA*)out, o_sh, o_st, H, rank, dr, page, window,
            scale);
  return ix_launch_status();
}

// q_lat: element (h, t, d) at h * ql_sh + t * ql_st + d, d < rank; q_rot: [T, H, dr];
// cache: [pages * page, rank + dr]; out: element (h, t, d) at h * o_sh + t * o_st + d.
IX_API int ix_latent_attention(const void* q_lat, long long ql_sh, long long ql_st,
                               const void* q_rot, const void* cache, const int* block_table,
                               int max_blocks, const int* seq_of_token, const int* positions,
                               void* out, long long o_sh, long long o_st, int act_dtype, int T,
                               int H, int rank, int dr, int page, int window, float scale,
                               cudaStream_t stream) {
  if (T <= 0) return IX_OK;
  if (H <= 0 || H > 65535 * LA_HB || rank <= 0 || rank > 1024 || dr < 0 || page <= 0 ||
      max_blocks <= 0)
    return IX_ERR_SIZE;
#define IX_LA(NR)                                                                               \
  IX_DISPATCH_DTYPE(act_dtype, TA,                                                              \
                    return (launch_latent_attention<TA, NR>(                                    \
                        q_lat, ql_sh, ql_st, q_rot, cache, block_table, max_blocks, seq_of_token, \
                        positions, out, o_sh, o_st, T, H, rank, dr, page, window, scale, stream)))
  if (rank <= 128) IX_LA(4);
  else if (rank <= 256) IX_LA(8);
  else if (rank <= 512) IX_LA(16);
  else IX_LA(32);
#undef IX_LA
  return IX_ERR_SIZE;
}
