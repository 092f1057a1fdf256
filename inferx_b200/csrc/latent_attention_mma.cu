// Tensor-core form of attention over cached latent records (see latent_attention.cu for
// what is computed): bfloat16, latent sizes 64, 128, 256 or 512, a rotated part that is a
// multiple of 16.  One kernel for prompts, portions and single tokens.
//
// A block owns 64 rows (16 in steps of single tokens with few heads), a row being one (token, head) pair of one sequence, tokens
// outermost: all heads of a token share the token's keys, and neighbouring tokens share
// all but one, so the 64 rows walk one run of key tiles.  Keys come in tiles of 32 that
// start on multiples of 32 of the absolute position; a row's masked keys weigh exactly
// nothing, so a row's result depends on its own keys only, not on its neighbours in the
// block or the batch.
//
// Per key tile (cp.async, two buffers; records of keys outside the tile's reach are
// zero-filled), with the warps arranged as 4 row groups x NSPLIT:
//   1. scores: warp (rg, cg) multiplies its 16 rows with all 32 keys over every NSPLIT-th
//      slice of 16 record entries (mma.sync m16n8k16, fp32 accumulation) and leaves its
//      partial sums in shared memory as fp32;
//   2. softmax: the warp adds the partial sums (in a fixed order) of its 16 / NSPLIT rows,
//      masks each row by its own window, updates the row's running maximum and sum (fp32,
//      exp2) and leaves the weights as bf16 and the row's rescaling factor in shared memory;
//   3. values: the warp multiplies the weights of its 16 rows with its CW columns of the
//      latents (the first `rank` entries of the same records, read transposed),
//      CW = rank / NSPLIT <= 128 columns a warp, accumulators in registers.
//
// When few blocks would run over long runs of keys (single tokens late in long sequences),
// the keys are cut into chunks of `chunk_tiles` tiles that start on multiples of the chunk
// in absolute position; blockIdx.y picks the chunk, partial results (unnormalised output,
// maximum, sum) go to scratch, and a second kernel merges them in chunk order.
#include "common.cuh"

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

#define LM_PLD 40   // bf16 per row of weights: 32 + 8 (80 bytes: an odd number of 16-byte units)

template <int CW, int NSPLIT, int RG>
__global__ void __launch_bounds__(32 * RG * NSPLIT)
latent_attention_mma_kernel(const bf16* __restrict__ q_lat, long long ql_sh, long long ql_st,
                            const bf16* __restrict__ q_rot, const bf16* __restrict__ cache,
                            const int* __restrict__ block_table, int max_blocks,
                            const int* __restrict__ cu_q, const int* __restrict__ q_pos0, int S,
                            bf16* __restrict__ out, long long o_sh, long long o_st, int H, int dr,
                            int page, int window, float scale_log2, int tokens_per_tile,
                            int heads_per_tile, int head_groups, int ld, int chunk_tiles,
                            float* __restrict__ part_o, float* __restrict__ part_ml) {
  constexpr int RANK = CW * NSPLIT;
  constexpr int NTHREADS = 32 * RG * NSPLIT;
  constexpr int LM_ROWS = 16 * RG;         // (token, head) rows of the block
  constexpr int RPW = 16 / NSPLIT;         // rows whose softmax a warp owns
  constexpr int LPR = 32 / RPW;            // lanes per such row
  constexpr int CPL = 32 / LPR;            // keys per lane
  constexpr bool PIPELINED = NSPLIT < 4;
  extern __shared__ __align__(16) unsigned char lm_smem[];
  IX_PDL_WAIT();
  const int Dk = RANK + dr;
  bf16* Qs = reinterpret_cast<bf16*>(lm_smem);                       // [64][ld]
  bf16* Ks = Qs + LM_ROWS * ld;                                      // [2][32][ld]
  float* Sp = reinterpret_cast<float*>(Ks + 2 * LM_KT * ld);         // [NSPLIT][64][LM_SLD]
  bf16* Ps = reinterpret_cast<bf16*>(Sp + NSPLIT * LM_ROWS * LM_SLD);  // [64][LM_PLD]
  float* corr_s = reinterpret_cast<float*>(Ps + LM_ROWS * LM_PLD);   // [64]
  float* m_s = corr_s + LM_ROWS;                                     // [64] (at the end)
  float* l_s = m_s + LM_ROWS;                                        // [64] (at the end)

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
  const int tok0 = (bt - before) * tokens_per_tile;    // first token of the tile within this step's portion
  const int ntok = min(tokens_per_tile, q_len - tok0);
  const int first_pos = q_pos0[s] + tok0;
  const int last_pos = first_pos + ntok - 1;
  const int* table = block_table + (size_t)s * max_blocks;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp % RG, cg = warp / RG;
  const int g = lane >> 2, t4 = lane & 3;
  const int cpr = Dk >> 3;                                           // 16-byte chunks per record
  const int nsplit_out = gridDim.y;

  const int lo_first = window > 0 ? max(0, first_pos - window + 1) : 0;
  int tile_lo = lo_first / LM_KT, tile_hi = last_pos / LM_KT;        // absolute tile indices
  if (chunk_tiles > 0) {
    const int c = tile_lo / chunk_tiles + blockIdx.y;
    tile_lo = max(tile_lo, c * chunk_tiles);
    tile_hi = min(tile_hi, c * chunk_tiles + chunk_tiles - 1);
  }
  const int ntiles = tile_hi - tile_lo + 1;
  if (ntiles <= 0) {
    // nothing of this chunk is in reach: an empty partial result
    for (int r = tid; r < LM_ROWS; r += NTHREADS) {
      const int tl = r / heads_per_tile, h = hg * heads_per_tile + (r - tl * heads_per_tile);
      if (tl < ntok && h < H) {
        float* ml = part_ml + (((size_t)(q0 + tok0 + tl) * H + h) * nsplit_out + blockIdx.y) * 2;
        ml[0] = -INFINITY;
        ml[1] = 0.f;
      }
    }
    return;
  }

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

  // Each thread copies a fixed share of one key's record, so a tile costs it one look-up
  // in the block table and no divisions.
  constexpr int TPR = NTHREADS / LM_KT;            // threads per key record
  const int key_j = tid / TPR, key_c0 = tid % TPR;
  auto load_keys = [&](int tile, int buf) {
    const int kp = (tile_lo + tile) * LM_KT + key_j;
    bool valid = kp >= lo_first && kp <= last_pos;
    const bf16* src = cache;
    if (valid) {
      const int pg = table[kp / page];
      valid = pg >= 0;
      if (valid) src = cache + ((size_t)pg * page + kp % page) * Dk;
    }
    bf16* dst = Ks + (buf * LM_KT + key_j) * ld;
    for (int cc = key_c0; cc < cpr; cc += TPR)
      lm_cp16(dst + cc * 8, valid ? src + cc * 8 : src, valid);
  };
  load_keys(0, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");

  // the row whose softmax this lane shares in
  const int srow = rg * 16 + cg * RPW + lane / LPR;
  const int scol = (lane % LPR) * CPL;
  int pos_s, lo_s;
  {
    const int tl = srow / heads_per_tile, h = hg * heads_per_tile + (srow - tl * heads_per_tile);
    const bool valid = tl < ntok && h < H;
    pos_s = valid ? first_pos + tl : -1;
    lo_s = valid ? (window > 0 ? max(0, pos_s - window + 1) : 0) : 0;
  }
  float m_run = -INFINITY, l_run = 0.f;
  float o[CW / 8][4];
#pragma unroll
  for (int n = 0; n < CW / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const int ksteps = Dk / 16;

  for (int tile = 0; tile < ntiles; ++tile) {
    const int buf = tile & 1;
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    if (tile + 1 < ntiles) load_keys(tile + 1, buf ^ 1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* Kb = Ks + buf * LM_KT * ld;
    const int k0 = (tile_lo + tile) * LM_KT;

    // 1. partial scores of 16 rows x 32 keys over this warp's slices of the record
    {
      float acc[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const bf16* qa = Qs + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8;
      const bf16* kb = Kb + ((lane & 7) + (lane >> 4) * 8) * ld + ((lane >> 3) & 1) * 8;
      // PIPELINED (set where the kernel is declared): fragments of the next slice are
      // fetched before the products of this one are issued.  With sixteen warps at the
      // 128-register limit that measured slower (137 against 148 TFLOP/s), with eight or
      // four warps faster (129 against 108).
      if constexpr (PIPELINED) {
        unsigned a[4], b[8];
        if (cg < ksteps) {
          lm_ldsm4(a[0], a[1], a[2], a[3], qa + cg * 16);
          lm_ldsm4(b[0], b[1], b[2], b[3], kb + cg * 16);
          lm_ldsm4(b[4], b[5], b[6], b[7], kb + 16 * ld + cg * 16);
        }
        for (int ks = cg; ks < ksteps; ks += NSPLIT) {
          unsigned an[4], bn[8];
          const int kn = ks + NSPLIT;
          if (kn < ksteps) {
            lm_ldsm4(an[0], an[1], an[2], an[3], qa + kn * 16);
            lm_ldsm4(bn[0], bn[1], bn[2], bn[3], kb + kn * 16);
            lm_ldsm4(bn[4], bn[5], bn[6], bn[7], kb + 16 * ld + kn * 16);
          }
          lm_mma(acc[0], a, b[0], b[1]);
          lm_mma(acc[1], a, b[2], b[3]);
          lm_mma(acc[2], a, b[4], b[5]);
          lm_mma(acc[3], a, b[6], b[7]);
          if (kn < ksteps) {
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = an[i];
#pragma unroll
            for (int i = 0; i < 8; ++i) b[i] = bn[i];
          }
        }
      } else {
        for (int ks = cg; ks < ksteps; ks += NSPLIT) {
          unsigned a[4], b0, b1, b2, b3;
          lm_ldsm4(a[0], a[1], a[2], a[3], qa + ks * 16);
          lm_ldsm4(b0, b1, b2, b3, kb + ks * 16);
          lm_mma(acc[0], a, b0, b1);
          lm_mma(acc[1], a, b2, b3);
          lm_ldsm4(b0, b1, b2, b3, kb + 16 * ld + ks * 16);
          lm_mma(acc[2], a, b0, b1);
          lm_mma(acc[3], a, b2, b3);
        }
      }
      float* d0 = Sp + (cg * LM_ROWS + rg * 16 + g) * LM_SLD + 2 * t4;
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        *reinterpret_cast<float2*>(d0 + n * 8) = make_float2(acc[n][0], acc[n][1]);
        *reinterpret_cast<float2*>(d0 + 8 * LM_SLD + n * 8) = make_float2(acc[n][2], acc[n][3]);
      }
    }
    __syncthreads();

    // 2. running softmax of this warp's own rows; weights and rescaling factors to shared memory
    {
      float sv[CPL];
      const float* src = Sp + srow * LM_SLD + scol;
#pragma unroll
      for (int c = 0; c < CPL; c += 4) {
        float4 v = *reinterpret_cast<const float4*>(src + c);
#pragma unroll
        for (int p = 1; p < NSPLIT; ++p) {
          const float4 w = *reinterpret_cast<const float4*>(src + p * LM_ROWS * LM_SLD + c);
          v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
        }
        sv[c] = v.x; sv[c + 1] = v.y; sv[c + 2] = v.z; sv[c + 3] = v.w;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        const int kp = k0 + scol + c;
        sv[c] = (kp >= lo_s && kp <= pos_s) ? sv[c] * scale_log2 : -INFINITY;
        mx = fmaxf(mx, sv[c]);
      }
#pragma unroll
      for (int d = 1; d < LPR; d <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
      const float m_new = fmaxf(m_run, mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = exp2f(m_run - m_use);
      float sum = 0.f;
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
        sv[c] = exp2f(sv[c] - m_use);
        sum += sv[c];
      }
#pragma unroll
      for (int d = 1; d < LPR; d <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
      l_run = l_run * corr + sum;
      m_run = m_new;
      bf16* pd = Ps + srow * LM_PLD + scol;
#pragma unroll
      for (int c = 0; c < CPL; c += 2)
        *reinterpret_cast<unsigned*>(pd + c) = lm_pack(sv[c], sv[c + 1]);
      if (lane % LPR == 0) corr_s[srow] = corr;
    }
    __syncthreads();

    // 3. weights x latents for this warp's 16 rows and CW columns
    {
      const float c0 = corr_s[rg * 16 + g], c1 = corr_s[rg * 16 + g + 8];
#pragma unroll
      for (int n = 0; n < CW / 8; ++n) {
        o[n][0] *= c0;
        o[n][1] *= c0;
        o[n][2] *= c1;
        o[n][3] *= c1;
      }
      const bf16* pa_src = Ps + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LM_PLD + (lane >> 4) * 8;
      const bf16* vb = Kb + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + cg * CW + (lane >> 4) * 8;
      if constexpr (PIPELINED) {
        unsigned pa[2][4];
        lm_ldsm4(pa[0][0], pa[0][1], pa[0][2], pa[0][3], pa_src);
        lm_ldsm4(pa[1][0], pa[1][1], pa[1][2], pa[1][3], pa_src + 16);
        // 2 x CW / 16 steps, each one 16 keys x 16 columns; the next step's latents are
        // fetched before this step's products are issued
        constexpr int STEPS = 2 * (CW / 16);
        unsigned vb0, vb1, vb2, vb3;
        lm_ldsm4t(vb0, vb1, vb2, vb3, vb);
#pragma unroll
        for (int st = 0; st < STEPS; ++st) {
          const int ks2 = st / (CW / 16), np = st % (CW / 16);
          unsigned n0 = 0, n1 = 0, n2 = 0, n3 = 0;
          if (st + 1 < STEPS) {
            const int ks2n = (st + 1) / (CW / 16), npn = (st + 1) % (CW / 16);
            lm_ldsm4t(n0, n1, n2, n3, vb + ks2n * 16 * ld + npn * 16);
          }
          lm_mma(o[2 * np], pa[ks2], vb0, vb1);
          lm_mma(o[2 * np + 1], pa[ks2], vb2, vb3);
          vb0 = n0; vb1 = n1; vb2 = n2; vb3 = n3;
        }
      } else {
#pragma unroll
        for (int ks2 = 0; ks2 < 2; ++ks2) {
          unsigned pa[4];
          lm_ldsm4(pa[0], pa[1], pa[2], pa[3], pa_src + ks2 * 16);
#pragma unroll
          for (int np = 0; np < CW / 16; ++np) {
            unsigned b0, b1, b2, b3;
            lm_ldsm4t(b0, b1, b2, b3, vb + ks2 * 16 * ld + np * 16);
            lm_mma(o[2 * np], pa, b0, b1);
            lm_mma(o[2 * np + 1], pa, b2, b3);
          }
        }
      }
    }
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  if (lane % LPR == 0) {
    m_s[srow] = m_run;
    l_s[srow] = l_run;
  }
  __syncthreads();

#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = rg * 16 + g + 8 * i;
    const int tl = r / heads_per_tile, h = hg * heads_per_tile + (r - tl * heads_per_tile);
    if (!(tl < ntok && h < H)) continue;
    const size_t tok = (size_t)(q0 + tok0 + tl);
    if (chunk_tiles > 0) {
      const size_t slot = (tok * H + h) * nsplit_out + blockIdx.y;
      float* dst = part_o + slot * RANK + cg * CW + 2 * t4;
#pragma unroll
      for (int n = 0; n < CW / 8; ++n)
        *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i], o[n][2 * i + 1]);
      if (cg == 0 && t4 == 0) {
        part_ml[slot * 2] = m_s[r];
        part_ml[slot * 2 + 1] = l_s[r];
      }
    } else {
      const float l = l_s[r];
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* dst = out + (size_t)h * o_sh + tok * o_st + cg * CW + 2 * t4;
#pragma unroll
      for (int n = 0; n < CW / 8; ++n)
        *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
            __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
  }
}

// Merge of the chunks' partial results, in chunk order: one block per (token, head).  The
// chunks' weights exp2(m_i - m) are formed once, in shared memory.
__global__ void latent_attention_merge_kernel(const float* __restrict__ part_o,
                                              const float* __restrict__ part_ml, int nsplit,
                                              bf16* __restrict__ out, long long o_sh,
                                              long long o_st, int H, int rank) {
  extern __shared__ float merge_w[];     // [nsplit]
  __shared__ float scratch[32];
  IX_PDL_WAIT();
  const int tok = blockIdx.x / H, h = blockIdx.x % H;
  const float* ml = part_ml + (size_t)blockIdx.x * nsplit * 2;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < nsplit; i += blockDim.x)
    if (ml[2 * i + 1] > 0.f) m = fmaxf(m, ml[2 * i]);
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = m;
  __syncthreads();
  m = -INFINITY;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, scratch[w]);
  for (int i = threadIdx.x; i < nsplit; i += blockDim.x)
    merge_w[i] = ml[2 * i + 1] > 0.f ? exp2f(ml[2 * i] - m) : 0.f;
  __syncthreads();
  float l = 0.f;
  for (int i = 0; i < nsplit; ++i) l += merge_w[i] * ml[2 * i + 1];    // chunk order
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  const float* po = part_o + (size_t)blockIdx.x * nsplit * rank;
  bf16* dst = out + (size_t)h * o_sh + (size_t)tok * o_st;
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int i = 0; i < nsplit; ++i) {
      const float w = merge_w[i];
      if (w > 0.f) acc += po[(size_t)i * rank + d] * w;   // an empty chunk's output was never written
    }
    dst[d] = __float2bfloat16_rn(acc * inv);
  }
}

// Whether the tensor-core form takes these sizes.
IX_API int ix_latent_attention_mma_applies(int rank, int dr) {
  return (rank == 64 || rank == 128 || rank == 256 || rank == 512) && dr >= 0 && dr % 16 == 0 &&
         dr <= 256;
}

// Tokens of a sequence that share a block of `rows` (16 or 64) (token, head) rows.
IX_API int ix_latent_attention_mma_tokens_per_tile(int H, int rows) {
  return H >= rows ? 1 : rows / H;
}

// How the keys are cut when few blocks face long runs of keys: *chunk_tiles tiles of 32
// keys a chunk (0: no cutting) and the number of chunks a block row needs.  `span` is the
// longest run of keys a block can meet.
IX_API int ix_latent_attention_mma_chunks(int blocks, int span, int* chunk_tiles) {
  *chunk_tiles = 0;
  const int tiles = (span + LM_KT - 1) / LM_KT + 1;
  if (blocks >= 148 || tiles < 16) return 1;
  int want = (2 * 148) / blocks;      // chunks that fill the device's block slots once, not more
  if (want < 2) return 1;
  int ct = (tiles + want - 1) / want;
  if (ct < 4) ct = 4;
  *chunk_tiles = ct;
  return (tiles + ct - 1) / ct + 1;
}

template <int CW, int NSPLIT, int RG>
static int launch_lm(const void* q_lat, long long ql_sh, long long ql_st, const void* q_rot,
                     const void* cache, const int* block_table, int max_blocks, const int* cu_q,
                     const int* q_pos0, int S, void* out, long long o_sh, long long o_st, int H,
                     int dr, int page, int window, float scale, int num_tiles, int chunk_tiles,
                     int nchunks, float* part_o, float* part_ml, cudaStream_t stream) {
  constexpr int LM_ROWS = 16 * RG;
  const int Dk = CW * NSPLIT + dr;
  const int ld = lm_ld(Dk);
  const size_t smem = (size_t)(LM_ROWS + 2 * LM_KT) * ld * sizeof(bf16) +
                      (size_t)NSPLIT * LM_ROWS * LM_SLD * sizeof(float) +
                      (size_t)LM_ROWS * LM_PLD * sizeof(bf16) + 3 * LM_ROWS * sizeof(float);
  if (smem > 227 * 1024) return IX_ERR_SMEM;
  auto kern = latent_attention_mma_kernel<CW, NSPLIT, RG>;
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
  ix_launch(kern, dim3(num_tiles * head_groups, chunk_tiles > 0 ? nchunks : 1),
            dim3(32 * RG * NSPLIT), smem, stream, (const bf16*)q_lat, ql_sh, ql_st,
            (const bf16*)q_rot, (const bf16*)cache, block_table, max_blocks, cu_q, q_pos0, S,
            (bf16*)out, o_sh, o_st, H, dr, page, window, scale * 1.4426950408889634f, tpt, hpt,
            head_groups, ld, chunk_tiles, part_o, part_ml);
  return ix_launch_status();
}

// rows: 64 (four groups of 16 rows a block) or 16 (one group: steps of single tokens with
// few heads, where the larger block would be mostly empty rows).
// num_tiles = sum over sequences of ceil(q_len / tokens_per_tile).  All tensors bf16; q_lat
// rows, q_rot rows and cache records must start on 16-byte boundaries.  With chunk_tiles >
// 0 the keys are cut (see ix_latent_attention_mma_chunks): part_o [T, H, nchunks, rank] and
// part_ml [T, H, nchunks, 2] fp32 are scratch, and the merge kernel follows.
IX_API int ix_latent_attention_mma(const void* q_lat, long long ql_sh, long long ql_st,
                                   const void* q_rot, const void* cache, const int* block_table,
                                   int max_blocks, const int* cu_q, const int* q_pos0, int S,
                                   void* out, long long o_sh, long long o_st, int T, int H,
                                   int rank, int dr, int page, int window, float scale,
                                   int num_tiles, int rows, int chunk_tiles, int nchunks,
                                   float* part_o, float* part_ml, cudaStream_t stream) {
  if (num_tiles <= 0 || S <= 0) return IX_OK;
  if (rows != 16 && rows != 64) return IX_ERR_SIZE;
  if (!ix_latent_attention_mma_applies(rank, dr) || H <= 0 || page <= 0 || max_blocks <= 0)
    return IX_ERR_SIZE;
  if (chunk_tiles > 0 && (nchunks <= 0 || nchunks > 65535 || !part_o || !part_ml))
    return IX_ERR_SIZE;
  if ((((uintptr_t)q_lat | (uintptr_t)q_rot | (uintptr_t)cache | (uintptr_t)out) & 15) ||
      (ql_sh % 8) || (ql_st % 8) || (o_sh % 2) || (o_st % 2))
    return IX_ERR_ALIGN;
  int code;
#define IX_LM1(CW, NS, RG)                                                                       \
  code = launch_lm<CW, NS, RG>(q_lat, ql_sh, ql_st, q_rot, cache, block_table, max_blocks, cu_q, \
                               q_pos0, S, out, o_sh, o_st, H, dr, page, window, scale,           \
                               num_tiles, chunk_tiles, nchunks, part_o, part_ml, stream)
#define IX_LM(CW, NS)            \
  do {                           \
    if (rows == 16) {            \
      IX_LM1(CW, NS, 1);         \
    } else {                     \
      IX_LM1(CW, NS, 4);         \
    }                            \
  } while (0)
  if (rank == 64) IX_LM(64, 1);
  else if (rank == 128) IX_LM(128, 1);
  else if (rank == 256) IX_LM(128, 2);
  else IX_LM(128, 4);
#undef IX_LM
#undef IX_LM1
  if (code != IX_OK || chunk_tiles <= 0) return code;
  ix_launch(latent_attention_merge_kernel, dim3(T * H), dim3(rank >= 256 ? 256 : 128),
            (size_t)nchunks * sizeof(float), stream,
            (const float*)part_o, (const float*)part_ml, nchunks, (bf16*)out, o_sh, o_st, H, rank);
  return ix_launch_status();
}
