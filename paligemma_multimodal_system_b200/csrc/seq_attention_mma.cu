// Causal attention of prompt portions over the paged bf16 cache on the tensor cores, with the probabilities kept at fp32
// precision.
//
// The design asks for scores and probabilities in 32 bits.  q and k are bf16 here (they are stored so), so S = Q K^T from
// bf16 x bf16 products accumulated in fp32 is exact to fp32 rounding.  The probabilities P = exp(s - m) stay fp32 in
// registers; for P V each is cut into THREE bf16 terms p = p1 + p2 + p3 (8 + 8 + 8 mantissa bits) and the product is three
// tensor-core passes over the same bf16 V tile accumulated in fp32 -- the result carries fp32 P, not a bf16 rounding of it.
// Soft cap, running max / sum and the output gate are fp32 SIMT code on the accumulator fragments.
//
// CTA = 64 query rows (token x query head of one k/v head) of one entry, 4 warps x 16 rows; keys in tiles of 64.
// mma.sync.m16n8k16 fragments: S accumulators of two adjacent 8-key blocks are, element for element, the A operand of one
// 16-key step of P V, so P never leaves the registers.  (tcgen05 would want P in shared or tensor memory as bf16; three
// passes from there cost the round trips this kernel avoids.)
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

namespace {

__device__ __forceinline__ void mma16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// four 8 x 8 bf16 matrices from shared memory, transposed: key-major value rows -> the k-pairs an m16n8k16 B fragment wants
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* p) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}

// 16-byte asynchronous copy global -> shared (cp.async group semantics)
__device__ __forceinline__ void cp_async16(bf16* smem_dst, const bf16* gmem_src) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem_src) : "memory");
}

// tanh to fp32 accuracy without the library's slow path: odd series below 0.1 (next term 17 x^7 / 315 < 6e-10), else
// 1 - 2 / (exp(2|x|) + 1), whose absolute error of ~1e-7 is relative there as well
__device__ __forceinline__ float tanh32(float x) {
  const float ax = fabsf(x), x2 = x * x;
  const float small = x * fmaf(x2, fmaf(x2, 0.13333333f, -0.33333334f), 1.0f);
  const float big = copysignf(1.0f - __fdividef(2.0f, exp2f(ax * 2.885390082f) + 1.0f), x);
  return ax < 0.1f ? small : big;
}

// p = hi + mid + lo with bf16 terms (round to nearest each time; the remainders are exact in fp32)
__device__ __forceinline__ void split3(float p, float q, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(p, q);
  const float2 hf = __bfloat1622float2(h);
  const float rp = p - hf.x, rq = q - hf.y;
  const __nv_bfloat162 m = __floats2bfloat162_rn(rp, rq);
  const float2 mf = __bfloat1622float2(m);
  const __nv_bfloat162 l = __floats2bfloat162_rn(rp - mf.x, rq - mf.y);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  mid = *reinterpret_cast<const uint32_t*>(&m);
  lo = *reinterpret_cast<const uint32_t*>(&l);
}

template <int DIM, int VDIM>
__global__ void __launch_bounds__(128, (DIM + VDIM <= 128) ? 4 : 2) attn_ragged_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                                                              const bf16* __restrict__ gate, long long ldg, bf16* __restrict__ out,
                                                              const int* __restrict__ entry_row0, const int* __restrict__ entry_n,
                                                              const int* __restrict__ entry_ctx, const int* __restrict__ page_table, int max_pages,
                                                              int page, int H, int G, float scale, float softcap, int skip_single, int gate_per_head,
                                                              PgAttnScore sx) {
  constexpr int KS = DIM / 16, NV = VDIM / 8, QP = DIM + 8, VLD = VDIM + 8;
  static_assert(VDIM % 16 == 0, "value blocks are fetched in pairs");
  const int e = blockIdx.z, g = blockIdx.y, gsz = H / G;
  const int n = entry_n[e], ctx = entry_ctx[e], row0 = entry_row0[e];
  if (skip_single && n == 1) return;
  const int rows = n * gsz;
  const int r0 = blockIdx.x * 64;
  if (r0 >= rows) return;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);  // [64][QP]
  bf16* Kb = Qs + 64 * QP;                    // two key tiles [64][QP]
  bf16* Vb = Kb + 2 * 64 * QP;                // two value tiles [64][VLD], key-major (P V reads them through ldmatrix.trans)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  // Q tile (zero rows past the end)
  for (int id = threadIdx.x; id < 64 * (DIM / 8); id += 128) {
    const int r = id / (DIM / 8), cc = id % (DIM / 8), rr = r0 + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (rr < rows) v = *reinterpret_cast<const uint4*>(q + (long long)(row0 + rr / gsz) * ((long long)H * DIM) + (long long)(g * gsz + rr % gsz) * DIM + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * QP + cc * 8) = v;
  }
  __syncthreads();
  uint32_t qa[KS][4];
  const int rl = warp * 16 + gq, rh = rl + 8;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(Qs + rl * QP + ks * 16 + 2 * tq);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(Qs + rh * QP + ks * 16 + 2 * tq);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(Qs + rl * QP + ks * 16 + 8 + 2 * tq);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(Qs + rh * QP + ks * 16 + 8 + 2 * tq);
  }
  const int lim_l = r0 + rl < rows ? ctx + (r0 + rl) / gsz : -1;  // last visible key of the lane's two rows = their queries' positions
  const int lim_h = r0 + rh < rows ? ctx + (r0 + rh) / gsz : -1;
  const int wrow_last = min(rows - 1, r0 + warp * 16 + 15);
  const int wlim = r0 + warp * 16 < rows ? ctx + wrow_last / gsz : -1;
  const int kmax = ctx + (min(rows, r0 + 64) - 1) / gsz;
  // optional parts of the score: window with kept first keys, per-head multiplier, logarithmic distance penalty
  const int window = sx.window > 0 ? sx.window : 0x3fffffff, keep = sx.window > 0 ? max(sx.keep_first, 0) : 0;
  const int head_l = g * gsz + (r0 + rl < rows ? (r0 + rl) % gsz : 0), head_h = g * gsz + (r0 + rh < rows ? (r0 + rh) % gsz : 0);
  const float sc_l = scale * (sx.head_scale != nullptr ? sx.head_scale[head_l] : 1.f), sc_h = scale * (sx.head_scale != nullptr ? sx.head_scale[head_h] : 1.f);
  const bool dist = sx.dist_a != nullptr;
  const float da_l = dist ? sx.dist_a[head_l] : 0.f, da_h = dist ? sx.dist_a[head_h] : 0.f;
  const float db_l = dist ? sx.dist_b[head_l] : 0.f, db_h = dist ? sx.dist_b[head_h] : 0.f;
  // key tiles wholly between the kept first keys and the first key inside the window of the CTA's first row are skipped
  const int keep_end = (keep + 63) & ~63;
  const int cta_lo = max(0, ctx + r0 / gsz - window + 1) & ~63;
  const int warp_lo = ctx + min(r0 + warp * 16, rows - 1) / gsz - window + 1;
  auto next_tile = [&](int k) {
    const int nx = k + 64;
    return (nx >= keep_end && nx < cta_lo) ? cta_lo : nx;
  };
  float oacc[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_l = -INFINITY, m_h = -INFINITY, l_l = 0.f, l_h = 0.f;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const int* pt = page_table + (long long)e * max_pages;
  const long long krow = (long long)G * DIM, vrow = (long long)G * VDIM;
  // K / V tiles go through two buffers: the next tile is in flight (cp.async) while this one is multiplied; rows past the last
  // key any row of the CTA sees are zero (a masked probability times a stale value must stay zero)
  auto fetch = [&](int k0, int buf) {
    bf16* Kd = Kb + buf * 64 * QP;
    bf16* Vd = Vb + buf * 64 * VLD;
    for (int id = threadIdx.x; id < 64 * (DIM / 8); id += 128) {
      const int r = id / (DIM / 8), cc = id % (DIM / 8), j = k0 + r;
      bf16* d = Kd + r * QP + cc * 8;
      if (j <= kmax) cp_async16(d, k_pages + ((long long)pt[j / page] * page + j % page) * krow + (long long)g * DIM + cc * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    for (int id = threadIdx.x; id < 64 * (VDIM / 8); id += 128) {
      const int r = id / (VDIM / 8), cc = id % (VDIM / 8), j = k0 + r;
      bf16* d = Vd + r * VLD + cc * 8;
      if (j <= kmax) cp_async16(d, v_pages + ((long long)pt[j / page] * page + j % page) * vrow + (long long)g * VDIM + cc * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
  };
  const int lm_key = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;  // this lane's row of a 16-key x 16-column block
  int cur = 0;
  const int k_first = next_tile(-64);
  fetch(k_first, 0);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int k0 = k_first; k0 <= kmax; k0 = next_tile(k0), cur ^= 1) {
    if (next_tile(k0) <= kmax) fetch(next_tile(k0), cur ^ 1);  // that buffer was released by the barrier at the end of the last iteration
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    __syncthreads();
    const bf16* Ks = Kb + cur * 64 * QP;
    const bf16* Vs = Vb + cur * 64 * VLD;
    if (k0 <= wlim && !(k0 >= keep && k0 + 64 <= warp_lo)) {  // else: no row of this warp sees a key of the tile
    float sacc[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * QP + ks * 16 + 2 * tq);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * QP + ks * 16 + 8 + 2 * tq);
        mma16816(sacc[nb], qa[ks], b0, b1);
      }
    }
    // scores -> probabilities (fp32), running max / sum per row; the four lanes of a quad share a row
    float mx_l = -INFINITY, mx_h = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float sc = sacc[nb][c] * ((c & 2) ? sc_h : sc_l);
        if (softcap > 0.f) sc = softcap * tanh32(sc * inv_cap);
        const int key = k0 + nb * 8 + 2 * tq + (c & 1);
        const int away = ((c & 2) ? lim_h : lim_l) - key;
        const bool vis = away >= 0 && (away < window || key < keep);
        if (dist && vis) sc -= ((c & 2) ? da_h : da_l) * log1pf(((c & 2) ? db_h : db_l) * (float)away);
        sc *= 1.4426950408889634f;  // base-2 exponentials below
        sc = vis ? sc : -INFINITY;
        sacc[nb][c] = sc;
        if (c & 2) mx_h = fmaxf(mx_h, sc); else mx_l = fmaxf(mx_l, sc);
      }
    mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 1)); mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 2));
    mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 1)); mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 2));
    const float mn_l = fmaxf(m_l, mx_l), mn_h = fmaxf(m_h, mx_h);
    const float ml_safe = mn_l > -INFINITY ? mn_l : 0.f, mh_safe = mn_h > -INFINITY ? mn_h : 0.f;  // rows that see no key yet
    const float corr_l = exp2f(m_l - ml_safe), corr_h = exp2f(m_h - mh_safe);
    float sum_l = 0.f, sum_h = 0.f;
#pragma unroll
    for (int nb = 0; nb < 8; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(sacc[nb][c] - ((c & 2) ? mh_safe : ml_safe));  // exp2(-inf) = 0 for masked keys
        sacc[nb][c] = p;
        if (c & 2) sum_h += p; else sum_l += p;
      }
    l_l = l_l * corr_l + sum_l;  // per-lane partial sums; the quad is added up at the end
    l_h = l_h * corr_h + sum_h;
    m_l = mn_l;
    m_h = mn_h;
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
      oacc[nv][0] *= corr_l; oacc[nv][1] *= corr_l; oacc[nv][2] *= corr_h; oacc[nv][3] *= corr_h;
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a1[4], a2[4], a3[4];
      split3(sacc[2 * kk][0], sacc[2 * kk][1], a1[0], a2[0], a3[0]);
      split3(sacc[2 * kk][2], sacc[2 * kk][3], a1[1], a2[1], a3[1]);
      split3(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], a1[2], a2[2], a3[2]);
      split3(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], a1[3], a2[3], a3[3]);
      const bf16* vbase = Vs + (kk * 16 + lm_key) * VLD + lm_col;
#pragma unroll
      for (int np = 0; np < NV / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vbase + np * 16);
        mma16816(oacc[2 * np], a1, b0, b1);
        mma16816(oacc[2 * np], a2, b0, b1);
        mma16816(oacc[2 * np], a3, b0, b1);
        mma16816(oacc[2 * np + 1], a1, b2, b3);
        mma16816(oacc[2 * np + 1], a2, b2, b3);
        mma16816(oacc[2 * np + 1], a3, b2, b3);
      }
    }
    }
    __syncthreads();  // every warp is done with this buffer before the next iteration refills it
  }
  l_l += __shfl_xor_sync(0xffffffffu, l_l, 1); l_l += __shfl_xor_sync(0xffffffffu, l_l, 2);
  l_h += __shfl_xor_sync(0xffffffffu, l_h, 1); l_h += __shfl_xor_sync(0xffffffffu, l_h, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int rr = r0 + (half ? rh : rl);
    if (rr >= rows) continue;
    const long long t = row0 + rr / gsz;
    const int head = g * gsz + rr % gsz;
    float lsum = half ? l_h : l_l, osc = 1.f;
    if (sx.sink != nullptr) {  // the sink joins the denominator once (m is in base-2 units)
      const float mrow = half ? m_h : m_l, sk = sx.sink[head] * 1.4426950408889634f, mm = fmaxf(mrow, sk);
      osc = exp2f(mrow - mm);
      lsum = lsum * osc + exp2f(sk - mm);
    }
    const float inv = osc / lsum;
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
      const int col = nv * 8 + 2 * tq;
      float v0 = oacc[nv][2 * half] * inv, v1 = oacc[nv][2 * half + 1] * inv;
      if (gate != nullptr) {
        float2 gg;
        if (gate_per_head) gg.x = gg.y = __bfloat162float(gate[t * ldg + head]);  // one scalar gate per head
        else gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(gate + t * ldg + (long long)head * VDIM + col));
        v0 *= 1.0f / (1.0f + expf(-gg.x));
        v1 *= 1.0f / (1.0f + expf(-gg.y));
      }
      *reinterpret_cast<__nv_bfloat162*>(out + t * ((long long)H * VDIM) + (long long)head * VDIM + col) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Decoded tokens of a latent-attention layer in the absorbed form, on the tensor cores.  The cache holds ONE row per token
// ([latent | rotated part], DIM wide) that is the key of every head and, in its first VDIM columns, the value: all H query heads of
// a token are the rows of one tile against the same keys, so the tile is read once for all heads.
//
// CTA = (key split, block of up to 64 heads, entry); warp = 16 heads.  Keys pass in tiles of 64 rows through two shared-memory
// buffers, row-major, the next tile in flight (cp.async) while the current one is multiplied.  S = Q K^T as in the kernel above (the Q fragments are re-read from shared memory per k step: DIM is up to 288).
// P V takes its B operand from the SAME tile with ldmatrix.trans (key-major rows -> the k-pairs an m16n8k16 B fragment wants),
// so the values are neither stored nor fetched separately; probabilities stay fp32 and enter as three bf16 terms.
// With several key splits the (max, sum, accumulator) triples go to `partial` in the layout of pg_attn_decode and its merge
// kernel finishes the rows.  VS > 1: the value columns are shared out over VS CTAs (each recomputes the scores; a thread's accumulators
// stay at 128 registers for value parts up to 512 wide).
// ---------------------------------------------------------------------------------------------------------------------
template <int DIM, int VDIM, int KT, int VS>
__global__ void __launch_bounds__(128) attn_latent_decode_mma_kernel(const bf16* __restrict__ q, const bf16* __restrict__ pages,
                                                                     const bf16* __restrict__ gate, long long ldg, bf16* __restrict__ out,
                                                                     float* __restrict__ partial, const int* __restrict__ entry_row0,
                                                                     const int* __restrict__ entry_n, const int* __restrict__ entry_ctx,
                                                                     const int* __restrict__ page_table, int max_pages, int page, int H, float scale, int window) {
  constexpr int VPART = VDIM / VS, KS = DIM / 16, NV = VPART / 8, LD = DIM + 8;
  static_assert(DIM % 16 == 0 && VDIM % VS == 0 && VPART % 16 == 0 && VDIM <= DIM && (KT == 32 || KT == 64), "tile shapes");
  constexpr int NB = KT / 8;  // 8-key blocks per tile
  const int e = blockIdx.z, h0 = (blockIdx.y / VS) * 64, v0 = (blockIdx.y % VS) * VPART, split = blockIdx.x, nsplit = gridDim.x;
  if (entry_n[e] != 1) return;
  const int ctx = entry_ctx[e];
  const long long t = entry_row0[e];
  const int nrows = (blockDim.x >> 5) * 16;
  extern __shared__ __align__(16) unsigned char smraw[];
  bf16* Qs = reinterpret_cast<bf16*>(smraw);  // [nrows][LD]
  bf16* Kbuf = Qs + nrows * LD;               // two key tiles [KT][LD]: the next one is fetched (cp.async) while this one is used
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  for (int id = threadIdx.x; id < nrows * (DIM / 8); id += blockDim.x) {
    const int r = id / (DIM / 8), cc = id % (DIM / 8);
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h0 + r < H) v = *reinterpret_cast<const uint4*>(q + (t * H + h0 + r) * DIM + cc * 8);
    *reinterpret_cast<uint4*>(Qs + r * LD + cc * 8) = v;
  }
  const int rl = warp * 16 + gq, rh = rl + 8;
  float oacc[NV][4];
#pragma unroll
  for (int i = 0; i < NV; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  float m_l = -INFINITY, m_h = -INFINITY, l_l = 0.f, l_h = 0.f;
  const int* pt = page_table + (long long)e * max_pages;
  const int lo = window > 0 ? max(0, ctx + 1 - window) : 0;  // a sliding window: keys lo .. ctx
  const int tile0 = lo / KT, ntiles = ctx / KT + 1;           // tiles tile0 .. ntiles - 1 hold them
  const float sc2 = scale * 1.4426950408889634f;
  // lane's row address inside a 16-key x 16-column block for ldmatrix.x4.trans: matrices (keys 0-7 | 8-15) x (columns 0-7 | 8-15)
  const int lm_key = (lane & 7) + ((lane >> 3) & 1) * 8, lm_col = (lane >> 4) * 8;
  auto fetch_tile = [&](int it, bf16* dst) {
    const int k0 = it * KT;
    for (int id = threadIdx.x; id < KT * (DIM / 8); id += blockDim.x) {
      const int r = id / (DIM / 8), cc = id % (DIM / 8), j = k0 + r;
      bf16* d = dst + r * LD + cc * 8;
      if (j <= ctx) cp_async16(d, pages + ((long long)pt[j / page] * page + j % page) * DIM + cc * 8);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
  };
  int cur = 0;
  if (tile0 + split < ntiles) fetch_tile(tile0 + split, Kbuf);
  asm volatile("cp.async.commit_group;" ::: "memory");
  for (int it = tile0 + split; it < ntiles; it += nsplit) {
    const int k0 = it * KT;
    const bf16* Ks = Kbuf + cur * KT * LD;
    if (it + nsplit < ntiles) fetch_tile(it + nsplit, Kbuf + (cur ^ 1) * KT * LD);  // that buffer was released by the barrier below
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 1;" ::: "memory");  // everything but the newest group has landed: this tile
    __syncthreads();
    float sacc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll 2
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(Qs + rl * LD + ks * 16 + 2 * tq);
      a[1] = *reinterpret_cast<const uint32_t*>(Qs + rh * LD + ks * 16 + 2 * tq);
      a[2] = *reinterpret_cast<const uint32_t*>(Qs + rl * LD + ks * 16 + 8 + 2 * tq);
      a[3] = *reinterpret_cast<const uint32_t*>(Qs + rh * LD + ks * 16 + 8 + 2 * tq);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * LD + ks * 16 + 2 * tq);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(Ks + (nb * 8 + gq) * LD + ks * 16 + 8 + 2 * tq);
        mma16816(sacc[nb], a, b0, b1);
      }
    }
    float mx_l = -INFINITY, mx_h = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = k0 + nb * 8 + 2 * tq + (c & 1);
        const float sc = (key <= ctx && key >= lo) ? sacc[nb][c] * sc2 : -INFINITY;
        sacc[nb][c] = sc;
        if (c & 2) mx_h = fmaxf(mx_h, sc); else mx_l = fmaxf(mx_l, sc);
      }
    mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 1)); mx_l = fmaxf(mx_l, __shfl_xor_sync(0xffffffffu, mx_l, 2));
    mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 1)); mx_h = fmaxf(mx_h, __shfl_xor_sync(0xffffffffu, mx_h, 2));
    const float mn_l = fmaxf(m_l, mx_l), mn_h = fmaxf(m_h, mx_h);  // finite: every tile of the loop holds a key in lo .. ctx, visible to every row
    const float corr_l = exp2f(m_l - mn_l), corr_h = exp2f(m_h - mn_h);
    float sum_l = 0.f, sum_h = 0.f;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float p = exp2f(sacc[nb][c] - ((c & 2) ? mn_h : mn_l));
        sacc[nb][c] = p;
        if (c & 2) sum_h += p; else sum_l += p;
      }
    l_l = l_l * corr_l + sum_l;
    l_h = l_h * corr_h + sum_h;
    m_l = mn_l;
    m_h = mn_h;
#pragma unroll
    for (int nv = 0; nv < NV; ++nv) {
      oacc[nv][0] *= corr_l; oacc[nv][1] *= corr_l; oacc[nv][2] *= corr_h; oacc[nv][3] *= corr_h;
    }
#pragma unroll
    for (int kk = 0; kk < KT / 16; ++kk) {
      uint32_t a1[4], a2[4], a3[4];
      split3(sacc[2 * kk][0], sacc[2 * kk][1], a1[0], a2[0], a3[0]);
      split3(sacc[2 * kk][2], sacc[2 * kk][3], a1[1], a2[1], a3[1]);
      split3(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1], a1[2], a2[2], a3[2]);
      split3(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3], a1[3], a2[3], a3[3]);
      const bf16* vbase = Ks + (kk * 16 + lm_key) * LD + lm_col + v0;
#pragma unroll
      for (int np = 0; np < NV / 2; ++np) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4_trans(b0, b1, b2, b3, vbase + np * 16);
        mma16816(oacc[2 * np], a1, b0, b1);
        mma16816(oacc[2 * np], a2, b0, b1);
        mma16816(oacc[2 * np], a3, b0, b1);
        mma16816(oacc[2 * np + 1], a1, b2, b3);
        mma16816(oacc[2 * np + 1], a2, b2, b3);
        mma16816(oacc[2 * np + 1], a3, b2, b3);
      }
    }
    __syncthreads();  // every warp is done with this buffer before the next iteration refills it
    cur ^= 1;
  }
  l_l += __shfl_xor_sync(0xffffffffu, l_l, 1); l_l += __shfl_xor_sync(0xffffffffu, l_l, 2);
  l_h += __shfl_xor_sync(0xffffffffu, l_h, 1); l_h += __shfl_xor_sync(0xffffffffu, l_h, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int head = h0 + (half ? rh : rl);
    if (head >= H) continue;
    const float lsum = half ? l_h : l_l, mrow = half ? m_h : m_l;
    if (nsplit == 1) {
      float g = 1.0f / lsum;
      if (gate != nullptr) g *= 1.0f / (1.0f + expf(-__bfloat162float(gate[t * ldg + head])));
#pragma unroll
      for (int nv = 0; nv < NV; ++nv)
        *reinterpret_cast<__nv_bfloat162*>(out + (t * H + head) * VDIM + v0 + nv * 8 + 2 * tq) =
            __floats2bfloat162_rn(oacc[nv][2 * half] * g, oacc[nv][2 * half + 1] * g);
    } else {
      float* pp = partial + (((long long)e * H + head) * nsplit + split) * (VDIM + 2);
      if (tq == 0 && v0 == 0) { pp[0] = mrow * 0.6931471805599453f; pp[1] = lsum; }  // the merge kernel works with natural exponentials
#pragma unroll
      for (int nv = 0; nv < NV; ++nv) {
        pp[2 + v0 + nv * 8 + 2 * tq] = oacc[nv][2 * half];
        pp[2 + v0 + nv * 8 + 2 * tq + 1] = oacc[nv][2 * half + 1];
      }
    }
  }
}

template <int DIM, int VDIM, int KT, int VS>
int launch_latent_kt(const void* q, const void* pages, const void* gate, long long ldg, void* out, float* partial, const int* row0, const int* n,
                     const int* ctx, const int* pt, int max_pages, int page, int entries, int nsplit, int H, float scale, int window, int warps, cudaStream_t st) {
  const size_t smem = ((size_t)(16 * warps + 2 * KT) * (DIM + 8)) * sizeof(bf16);
  auto kern = attn_latent_decode_mma_kernel<DIM, VDIM, KT, VS>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  kern<<<dim3(nsplit, ((H + 63) / 64) * VS, entries), 32 * warps, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(pages), static_cast<const bf16*>(gate),
                                                                      ldg, static_cast<bf16*>(out), partial, row0, n, ctx, pt, max_pages, page, H, scale, window);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

// up to 32 heads = two warps per CTA: 32-key tiles keep four such CTAs on an SM (shared memory), 64-key tiles only two; rows wider than
// 288 always take 32-key tiles (shared memory) and two CTAs per value half
template <int DIM, int VDIM>
int launch_latent(const void* q, const void* pages, const void* gate, long long ldg, void* out, float* partial, const int* row0, const int* n,
                  const int* ctx, const int* pt, int max_pages, int page, int entries, int nsplit, int H, float scale, int window, cudaStream_t st) {
  const int warps = H >= 64 ? 4 : (H + 15) / 16;
  constexpr int VS = VDIM > 256 ? 2 : 1;
  if (warps <= 2 || DIM > 288)
    return launch_latent_kt<DIM, VDIM, 32, VS>(q, pages, gate, ldg, out, partial, row0, n, ctx, pt, max_pages, page, entries, nsplit, H, scale, window, warps, st);
  return launch_latent_kt<DIM, VDIM, 64, VS>(q, pages, gate, ldg, out, partial, row0, n, ctx, pt, max_pages, page, entries, nsplit, H, scale, window, warps, st);
}

template <int DIM, int VDIM>
int launch(const void* q, const void* kp, const void* vp, const void* gate, long long ldg, void* out, const int* row0, const int* n, const int* ctx,
           const int* pt, int max_pages, int page, int entries, int max_n, int H, int G, float scale, float softcap, int skip_single, int gate_per_head,
           const PgAttnScore& sx, cudaStream_t st) {
  const size_t smem = ((size_t)3 * 64 * (DIM + 8) + (size_t)2 * 64 * (VDIM + 8)) * sizeof(bf16);
  auto kern = attn_ragged_mma_kernel<DIM, VDIM>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  dim3 grid((max_n * (H / G) + 63) / 64, G, entries);
  kern<<<grid, 128, smem, st>>>(static_cast<const bf16*>(q), static_cast<const bf16*>(kp), static_cast<const bf16*>(vp), static_cast<const bf16*>(gate), ldg,
                                static_cast<bf16*>(out), row0, n, ctx, pt, max_pages, page, H, G, scale, softcap, skip_single, gate_per_head, sx);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

}  // namespace

extern "C" int pg_attn_ragged_mma(const void* q, const void* k_pages, const void* v_pages, const void* gate, long long ldg, void* out,
                                  const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages, int page,
                                  int entries, int max_n, int H, int G, int dim, int vdim, float scale, float softcap, int skip_single, int gate_per_head,
                                  const PgAttnScore* score, void* stream) {
  if (entries <= 0 || max_n <= 0 || H <= 0 || G <= 0 || (H % G) != 0 || entries > 65535 || G > 65535) return PG_ERR_ARG;
  if (score != nullptr && ((score->dist_a == nullptr) != (score->dist_b == nullptr))) return PG_ERR_ARG;
  const PgAttnScore sx = score != nullptr ? *score : PgAttnScore{};
  // 16-byte row loads and bf16x2 gate / output accesses
  if (((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages) | reinterpret_cast<uintptr_t>(out)) & 15) ||
      (gate != nullptr && !gate_per_head && ((reinterpret_cast<uintptr_t>(gate) & 3) || (ldg & 1))))
    return PG_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define PG_MMA(D, V) \
  if (dim == D && vdim == V) \
    return launch<D, V>(q, k_pages, v_pages, gate, ldg, out, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, entries, max_n, H, G, scale, \
                        softcap, skip_single, gate_per_head, sx, st)
  PG_MMA(32, 32);
  PG_MMA(96, 64);    // explicit-head form of latent attention: [plain | rotated] keys
  PG_MMA(192, 128);
  PG_MMA(64, 64);
  PG_MMA(128, 128);
  PG_MMA(64, 128);
  PG_MMA(128, 64);
#undef PG_MMA
  return PG_ERR_ARG;  // other head sizes: pg_attn_ragged
}

extern "C" int pg_attn_latent_decode_mma(const void* q, const void* pages, const void* gate, long long ldg, void* out, float* partial,
                                         const int* entry_row0, const int* entry_n, const int* entry_ctx, const int* page_table, int max_pages,
                                         int page, int entries, int nsplit, int H, int dim, int vdim, float scale, int window, void* stream) {
  if (window < 0) return PG_ERR_ARG;
  if (entries <= 0 || entries > 65535 || nsplit <= 0 || nsplit > 64 || H <= 0 || page <= 0 || (nsplit > 1 && partial == nullptr)) return PG_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(pages) | reinterpret_cast<uintptr_t>(out)) & 15) return PG_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
#define PG_LAT(D, V) \
  if (dim == D && vdim == V) \
    return launch_latent<D, V>(q, pages, gate, ldg, out, partial, entry_row0, entry_n, entry_ctx, page_table, max_pages, page, entries, nsplit, H, scale, window, st)
  PG_LAT(96, 64);
  PG_LAT(160, 128);
  PG_LAT(192, 128);
  PG_LAT(288, 256);
  PG_LAT(544, 512);
  PG_LAT(576, 512);
#undef PG_LAT
  return PG_ERR_ARG;  // other row sizes: pg_attn_decode
}
