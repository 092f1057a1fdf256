// Tensor-core form of attention over cached latent records (see latent_attention.cu for
// what is computed): bfloat16, latent sizes 64, 128, 256 or 512, a rotated part that is a
// multiple of 16.  One kernel for prompts, portions and single tokens.
//
// A block owns 64 rows, a row being one (token, head) pair of one sequence, tokens
// outermost: all heads of a token share the token's keys, and neighbouring tokens share
// all but one, so the 64 rows walk one run of key tiles.  Keys come in tiles of 32 that
// start on multiples of 32 of the absolute position; a row's masked keys weigh exactly
// nothing, so a row's result depends on its own keys only, not on its neighbours in the
// block or the batch.
//
// Per key tile (cp.async, two buffers; records of keys outside the tile's reach are
// zero-filled):
//   1. scores: warp (rg, cg) of 4 x NSPLIT multiplies its 16 rows by its share of the 32
//      keys over the whole record (mma.sync m16n8k16, fp32 accumulation) and leaves the
//      scaled scores in shared memory as fp32;
//   2. every warp reads the 16 x 32 scores of its rows, masks by each row's own window,
//      updates the running maximum and sum (fp32, exp2), rounds the weights to bf16 and
//      multiplies them with its CW columns of the latents (the first `rank` entries of the
//      same records, read transposed), CW = rank / NSPLIT <= 128 columns a warp.
#include "common.cuh"

#define LM_ROWS 64
#define LM_KT 32
#define LM_SLD 40   // floats per score row: 32 + 8, so that rows g and g + 1..3 hit other banks

__device__ __forceinline__ void lm_cp16(void* smem, const void* gmem, bool valid) {
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void lm_ldsm4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                         const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void lm_ldsm2(unsigned& r0, unsigned& r1, const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r0), "=r"(r1)
               : "r"(a));
}
__device__ __forceinline__ void lm_ldsm4t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3,
                                          const void* p) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(a));
}
__device__ __forceinline__ void lm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned lm_pack(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

static inline int lm_ld(int dk) { return dk + (((dk / 8) % 2 == 0) ? 8 : 16); }

template <int CW, int NSPLIT>
__global__ void __launch_bounds__(128 * NSPLIT)
latent_attention_mma_kernel(const bf16* __restrict__ q_lat, long long ql_sh, long long ql_st,
                            const bf16* __restrict__ q_rot, const bf16* __restrict__ cache,
                            const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ cu_q, const int* __restrict__ q_pos0, int S,
                            bf16* __restrict__ out, long long o_sh, long long o_st, int H, int dr,
                            int page, int window, float scale_log2, int tokens_per_tile,
                            int heads_per_tile, int head_groups, int ld) {
  constexpr int RANK = CW * NSPLIT;
  constexpr int NT1 = 4 / NSPLIT;          // 8-key tiles of the scores a warp computes
  constexpr int NTHREADS = 128 * NSPLIT;
  extern __shared__ __align__(16) unsigned char lm_smem[];
  IX_PDL_WAIT();
  const int Dk = RANK + dr;
  bf16* Qs = reinterpret_cast<bf16*>(lm_smem);                       // [64][ld]
  bf16* Ks = Qs + LM_ROWS * ld;                                      // [2][32][ld]
  float* Ss = reinterpret_cast<float*>(Ks + 2 * LM_KT * ld);         // [2][64][LM_SLD]

  // which 64 rows: sequence, run of tokens, group of heads
  const int hg = blockIdx.x % head_groups;
  const int bt = blockIdx.x / head_groups;
  int s = 0, before = 0;
  for (; s < S; ++s) {
    const int n = (cu_q[s + 1] - cu_q[s] + tokens_per_tile - 1) / tokens_per_tile;
    if (bt < before + n) break;
    before += n;
  }
  if (s == S) return;
  const int q0 = cu_q[s], q_len = cu_q[s + 1] - q0;
  const int tok0 = (bt - before) * tokens_per_tile;            // first token of the tile, in the sequence's portion
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int first_pos = q_pos0[s] + tok0;
  const int last_pos = first_pos + ntok - 1;
  const int* table = block_table + (size_t)s * max_blocks;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp & 3, cg = warp >> 2;
  const int g = lane >> 2, t4 = lane & 3;
  const int cpr = Dk >> 3;                                           // 16-byte chunks per record

  // queries -> shared memory (rows without a token or a head are zeros)
  for (int c = tid; c < LM_ROWS * cpr; c += NTHREADS) {
    const int r = c / cpr, cc = c - r * cpr;
    const int tl = r / heads_per_tile, h = hg * heads_per_tile + (r - tl * heads_per_tile);
    const bool valid = tl < ntok && h < H;
    const bf16* src = q_lat;
    if (valid) {
      const size_t tok = (size_t)(q0 + tok0 + tl);
      src = cc * 8 < RANK ? q_lat + (size_t)h * ql_sh + tok * ql_st + cc * 8
                          : q_rot + (tok * H + h) * dr + (cc * 8 - RANK);
    }
    lm_cp16(Qs + r * ld + cc * 8, src, valid);
  }
  const int lo_first = window > 0 ? max(0, first_pos - window + 1) : 0;
  const int k_begin = (lo_first / LM_KT) * LM_KT;
  const int ntiles = (last_pos - k_begin) / LM_KT + 1;

  auto load_keys = [&](int tile, int buf) {
    const int k0 = k_begin + tile * LM_KT;
    bf16* dst = Ks + buf * LM_KT * ld;
    for (int c = tid; c < LM_KT * cpr; c += NTHREADS) {
      const int j = c / cpr, cc = c - j * cpr;
      const int kp = k0 + j;
      bool valid = kp >= lo_first && kp <= last_pos;
      const bf16* src = cache;
      if (valid) {
        const int pg = table[kp / page];
        valid = pg >= 0;
        if (valid) src = cache + ((size_t)pg * page + kp % page) * Dk + cc * 8;
      }
      lm_cp16(dst + j * ld + cc * 8, src, valid);
    }
  };
  load_keys(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // this thread's two rows (g and g + 8 of the warp's sixteen)
  int pos_r[2], lo_r[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rg * 16 + g + 8 * i;
    const int tl = r / heads_per_tile, h = hg * heads_per_tile + (r - tl * heads_per_tile);
    const bool valid = tl < ntok && h < H;
    pos_r[i] = valid ? first_pos + tl : -1;
    lo_r[i] = valid ? (window > 0 ? max(0, pos_r[i] - window + 1) : 0) : 0;
  }
  float m_r[2] = {-INFINITY, -INFINITY}, l_r[2] = {0.f, 0.f};
  float o[CW / 8][4];
#pragma unroll
  for (int n = 0; n < CW / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    if (tile + 1 < ntiles) load_keys(tile + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* Kb = Ks + buf * LM_KT * ld;
    float* Sb = Ss + buf * LM_ROWS * LM_SLD;
    const int k0 = k_begin + tile * LM_KT;

    // 1. scores of 16 rows x (32 / NSPLIT) keys
    {
      float acc[NT1][4];
#pragma unroll
      for (int n = 0; n < NT1; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const bf16* qa = Qs + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
      const int key_base = cg * 8 * NT1;
      const bf16* kb4 = Kb + (key_base + (lane & 7) + (lane >> 4) * 8) * ld + ((lane >> 3) & 1) * 8;
      const bf16* kb2 = Kb + (key_base + (lane & 7)) * ld + ((lane >> 3) & 1) * 8;
      for (int ks = 0; ks < Dk / 16; ++ks) {
        unsigned a[4];
        lm_ldsm4(a[0], a[1], a[2], a[3], qa + ks * 16);
        if (NT1 >= 2) {
#pragma unroll
          for (int np = 0; np < NT1 / 2; ++np) {
            unsigned b0, b1, b2, b3;
            lm_ldsm4(b0, b1, b2, b3, kb4 + np * 16 * ld + ks * 16);
            lm_mma(acc[2 * np], a, b0, b1);
            lm_mma(acc[2 * np + 1], a, b2, b3);
          }
        } else {
          unsigned b0, b1;
          lm_ldsm2(b0, b1, kb2 + ks * 16);
          lm_mma(acc[0], a, b0, b1);
        }
      }
#pragma unroll
      for (int n = 0; n < NT1; ++n) {
        float* d0 = Sb + (rg * 16 + g) * LM_SLD + key_base + n * 8 + 2 * t4;
        *reinterpret_cast<float2*>(d0) = make_float2(acc[n][0] * scale_log2, acc[n][1] * scale_log2);
        *reinterpret_cast<float2*>(d0 + 8 * LM_SLD) =
            make_float2(acc[n][2] * scale_log2, acc[n][3] * scale_log2);
      }
    }
    __syncthreads();

    // 2. running softmax of the warp's 16 rows over the tile's 32 keys, then weights x latents
    unsigned pa[2][4];
    float corr[2];
    {
      float sv[2][8];    // [row][16 * ks2 + {0,1} (+8: 2,3)] -> index ks2 * 4 + ...
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const float* srow = Sb + (rg * 16 + g + 8 * i) * LM_SLD + 2 * t4;
        float mx = -INFINITY;
#pragma unroll
        for (int q = 0; q < 4; ++q) {      // q: column block of 8 keys
          const float2 v = *reinterpret_cast<const float2*>(srow + q * 8);
          const int kp = k0 + q * 8 + 2 * t4;
          sv[i][2 * q] = (kp >= lo_r[i] && kp <= pos_r[i]) ? v.x : -INFINITY;
          sv[i][2 * q + 1] = (kp + 1 >= lo_r[i] && kp + 1 <= pos_r[i]) ? v.y : -INFINITY;
          mx = fmaxf(mx, fmaxf(sv[i][2 * q], sv[i][2 * q + 1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_r[i], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;
        corr[i] = exp2f(m_r[i] - m_use);
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          sv[i][q] = exp2f(sv[i][q] - m_use);
          sum += sv[i][q];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l_r[i] = l_r[i] * corr[i] + sum;
        m_r[i] = m_new;
      }
      // A fragments of the weights: keys 16 * ks2 + (0..7 | 8..15) are column blocks 2 ks2, 2 ks2 + 1
#pragma unroll
      for (int ks2 = 0; ks2 < 2; ++ks2) {
        pa[ks2][0] = lm_pack(sv[0][4 * ks2], sv[0][4 * ks2 + 1]);
        pa[ks2][1] = lm_pack(sv[1][4 * ks2], sv[1][4 * ks2 + 1]);
        pa[ks2][2] = lm_pack(sv[0][4 * ks2 + 2], sv[0][4 * ks2 + 3]);
        pa[ks2][3] = lm_pack(sv[1][4 * ks2 + 2], sv[1][4 * ks2 + 3]);
      }
    }
#pragma unroll
    for (int n = 0; n < CW / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
    const bf16* vb = Kb + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + cg * CW + (lane >> 4) * 8;
#pragma unroll
    for (int ks2 = 0; ks2 < 2; ++ks2) {
#pragma unroll
      for (int np = 0; np < CW / 16; ++np) {
        unsigned b0, b1, b2, b3;
        lm_ldsm4t(b0, b1, b2, b3, vb + ks2 * 16 * ld + np * 16);
        lm_mma(o[2 * np], pa[ks2], b0, b1);
        lm_mma(o[2 * np + 1], pa[ks2], b2, b3);
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    if (pos_r[i] < 0) continue;
    const int r = rg * 16 + g + 8 * i;
    const int tl = r / heads_per_tile, h = hg * heads_per_tile + (r - tl * heads_per_tile);
    const float inv = l_r[i] > 0.f ? 1.0f / l_r[i] : 0.f;
    bf16* dst = out + (size_t)h * o_sh + (size_t)(q0 + tok0 + tl) * o_st + cg * CW + 2 * t4;
#pragma unroll
    for (int n = 0; n < CW / 8; ++n)
      *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
          __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
  }
}

// Whether the tensor-core form takes these sizes.
IX_API int ix_latent_attention_mma_applies(int rank, int dr) {
  return (rank == 64 || rank == 128 || rank == 256 || rank == 512) && dr >= 0 && dr % 16 == 0 &&
         dr <= 256;
}

// Blocks the launch needs for sequences that bring q_lens[s] tokens each.
IX_API int ix_latent_attention_mma_tokens_per_tile(int H) {
  return H >= LM_ROWS ? 1 : LM_ROWS / H;
}

template <int CW, int NSPLIT>
static int launch_lm(const void* q_lat, long long ql_sh, long long ql_st, const void* q_rot,
                     const void* cache, const int* block_table, int max_blocks, const int* cu_q,
                     const int* q_pos0, int S, void* out, long long o_sh, long long o_st, int H,
                     int dr, int page, int window, float scale, int num_tiles,
                     cudaStream_t stream) {
  const int Dk = CW * NSPLIT + dr;
  const int ld = lm_ld(Dk);
  const size_t smem = (size_t)(LM_ROWS + 2 * LM_KT) * ld * sizeof(bf16) +
                      (size_t)2 * LM_ROWS * LM_SLD * sizeof(float);
  if (smem > 227 * 1024) return IX_ERR_SMEM;
  auto kern = latent_attention_mma_kernel<CW, NSPLIT>;
  static bool raised = false;     // per instantiation
  if (!raised) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  const int hpt = H >= LM_ROWS ? LM_ROWS : H;
  const int tpt = H >= LM_ROWS ? 1 : LM_ROWS / H;
  const int head_groups = (H + hpt - 1) / hpt;
  ix_launch(kern, dim3(num_tiles * head_groups), dim3(128 * NSPLIT), smem, stream,
            (const bf16*)q_lat, ql_sh, ql_st, (const bf16*)q_rot, (const bf16*)cache, block_table,
            max_blocks, cu_q, q_pos0, S, (bf16*)out, o_sh, o_st, H, dr, page, window,
            scale * 1.4426950408889634f, tpt, hpt, head_groups, ld);
  return ix_launch_status();
}

// num_tiles = sum over sequences of ceil(q_len / tokens_per_tile).  All tensors bf16; q_lat
// rows, q_rot rows and cache records must start on 16-byte boundaries.
IX_API int ix_latent_attention_mma(const void* q_lat, long long ql_sh, long long ql_st,
                                   const void* q_rot, const void* cache, const int* block_table,
                                   int max_blocks, const int* cu_q, const int* q_pos0, int S,
                                   void* out, long long o_sh, long long o_st, int H, int rank,
                                   int dr, int page, int window, float scale, int num_tiles,
                                   cudaStream_t stream) {
  if (num_tiles <= 0 || S <= 0) return IX_OK;
  if (!ix_latent_attention_mma_applies(rank, dr) || H <= 0 || page <= 0 || max_blocks <= 0)
    return IX_ERR_SIZE;
  if ((((uintptr_t)q_lat | (uintptr_t)q_rot | (uintptr_t)cache | (uintptr_t)out) & 15) ||
      (ql_sh % 8) || (ql_st % 8) || (o_sh % 2) || (o_st % 2))
    return IX_ERR_ALIGN;
#define IX_LM(CW, NS)                                                                          \
  return launch_lm<CW, NS>(q_lat, ql_sh, ql_st, q_rot, cache, block_table, max_blocks, cu_q,   \
                           q_pos0, S, out, o_sh, o_st, H, dr, page, window, scale, num_tiles,  \
                           stream)
  if (rank == 64) IX_LM(64, 1);
  if (rank == 128) IX_LM(128, 1);
  if (rank == 256) IX_LM(128, 2);
  IX_LM(128, 4);
#undef IX_LM
}
