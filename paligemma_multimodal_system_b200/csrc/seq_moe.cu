// Routed feed-forward (mixture of experts) of the token-sequence decoders, without a host round trip: the step may sit in a
// CUDA graph, so counts, offsets and tile lists stay on the device.
//
//   pg_moe_route     per token: softmax over the router outputs, choice score = probability + correction, optional group limit
//                    (experts in `group_count` equal runs of neighbours; only the `group_keep` runs with the largest best
//                    choice score stay eligible), the `top` largest choice scores, weights = chosen probabilities / their sum
//                    * scale.  Outputs >= n_real are identity experts.  Counts the (token, choice) pairs of every real expert.
//   pg_moe_plan      one CTA: expert offsets (exclusive scan), the list of row tiles (expert, first row, rows) and its length
//   pg_moe_scatter   pair -> its row in the expert-sorted order (and back)
//   pg_moe_gemm      out[row, f] = act(sum_k x[src(row), k] w[expert(row)][f, k]) over the tile list; plain fp32 FMAs, or
//                    mma.sync on the tensor cores for bf16 operands
//   pg_moe_combine   y[t] = sum_k weight[t, k] * (identity ? h[t] : expert_out[row(t, k)]) (+ shared[t])
//
// Router arithmetic, weights and the combine are fp32.
#include "common.cuh"
#include "paligemma_b200.h"

using bf16 = __nv_bfloat16;

#define PG_ST(s) reinterpret_cast<cudaStream_t>(s)
#define PG_RET()                                                    \
  do {                                                              \
    pg_count_launch(1);                                             \
    return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA; \
  } while (0)

namespace {

constexpr int MOE_TILE = 64;  // rows of one expert per GEMM tile

template <typename T>
__device__ __forceinline__ float ldm(const T* p, long long i);
template <>
__device__ __forceinline__ float ldm<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldm<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stm(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stm(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float wmaxf(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float wsumf(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// (value, index) of the largest value in the warp, lowest index among equals
__device__ __forceinline__ void wargmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

// One warp per token; probabilities and choice scores of the token in shared memory (2 * n_all floats per warp).
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, long long ld, const float* __restrict__ correction,
                                                        int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ counts, int T,
                                                        int n_all, int n_real, int top, int group_count, int group_keep, float scale,
                                                        const float* __restrict__ logit_bias) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= T) return;
  float* prob = sm + (size_t)warp * 2 * n_all;
  float* choice = prob + n_all;
  const float* z = logits + (long long)t * ld;
  float m = -INFINITY;
  for (int i = lane; i < n_all; i += 32) {
    const float zi = z[i] + (logit_bias != nullptr ? logit_bias[i] : 0.f);
    prob[i] = zi;
    m = fmaxf(m, zi);
  }
  m = wmaxf(m);
  float s = 0.f;
  for (int i = lane; i < n_all; i += 32) { const float e = expf(prob[i] - m); prob[i] = e; s += e; }
  s = wsumf(s);
  for (int i = lane; i < n_all; i += 32) {
    const float p = prob[i] / s;
    prob[i] = p;
    choice[i] = p + (correction != nullptr ? correction[i] : 0.f);
  }
  __syncwarp();
  if (group_count > 1 && group_keep < group_count) {
    // group g lives in lane g % 32, slot g / 32 (up to 8 slots = 256 groups): its score is its best choice score; group_keep rounds of
    // a warp arg-max mark the kept groups, the others get -inf choice scores (not 0: choice scores can be negative)
    const int per = n_all / group_count;
    float gs[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int g = lane + 32 * k;
      float b = -INFINITY;
      if (g < group_count)
        for (int i = 0; i < per; ++i) b = fmaxf(b, choice[g * per + i]);
      gs[k] = b;
    }
    unsigned keepmask[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // slot k kept (meaningful in the owning lane only)
    for (int r = 0; r < group_keep; ++r) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int g = lane + 32 * k;
        if (g < group_count && !(keepmask[k] & 1u) && (gs[k] > bv || (gs[k] == bv && g < bi))) { bv = gs[k]; bi = g; }
      }
      wargmax(bv, bi);
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (bi == lane + 32 * k) keepmask[k] |= 1u;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int g = lane + 32 * k;
      if (g < group_count && !(keepmask[k] & 1u))
        for (int i = 0; i < per; ++i) choice[g * per + i] = -INFINITY;
    }
    __syncwarp();
  }
  float wsum_sel = 0.f;
  int my_id = -1;
  float my_p = 0.f;
  for (int r = 0; r < top; ++r) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < n_all; i += 32) {
      const float c = choice[i];
      if (c > bv || (c == bv && i < bi)) { bv = c; bi = i; }
    }
    wargmax(bv, bi);
    if (bi >= n_all) bi = 0;  // every score -inf / NaN: never with finite inputs
    const float p = prob[bi];
    wsum_sel += p;
    if (lane == (r & 31)) { my_id = bi; my_p = p; }
    if (lane == 0) choice[bi] = -INFINITY;
    __syncwarp();
    if ((r & 31) == 31 || r == top - 1) {  // flush up to 32 choices
      const int base = r & ~31;
      if (my_id >= 0) {
        ids[(long long)t * top + base + lane] = my_id;
        weights[(long long)t * top + base + lane] = my_p;  // normalised below
        if (my_id < n_real) atomicAdd(counts + my_id, 1);
      }
      my_id = -1;
    }
  }
  __syncwarp();
  const float f = scale / (wsum_sel + 1e-20f);
  for (int r = lane; r < top; r += 32) weights[(long long)t * top + r] *= f;
}

// counts -> offsets, tile list.  plan[0] = number of tiles; tiles: (expert, first sorted row, rows) triples from plan[4].
__global__ void moe_plan_kernel(const int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ fill, int* __restrict__ plan, int n_real,
                                int max_tiles) {
  if (threadIdx.x != 0) return;
  int off = 0, nt = 0;
  for (int e = 0; e < n_real; ++e) {
    const int c = counts[e];
    offsets[e] = off;
    fill[e] = 0;
    for (int r = 0; r < c; r += MOE_TILE) {
      if (nt < max_tiles) {
        plan[4 + 3 * nt] = e;
        plan[4 + 3 * nt + 1] = off + r;
        plan[4 + 3 * nt + 2] = min(MOE_TILE, c - r);
      }
      ++nt;
    }
    off += c;
  }
  offsets[n_real] = off;
  plan[0] = nt < max_tiles ? nt : max_tiles;
}

__global__ void moe_scatter_kernel(const int* __restrict__ ids, const int* __restrict__ offsets, int* __restrict__ fill, int* __restrict__ sorted_pair,
                                   int* __restrict__ pair_row, int pairs, int n_real) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= pairs) return;
  const int e = ids[p];
  if (e >= n_real) { pair_row[p] = -1; return; }
  const int row = offsets[e] + atomicAdd(fill + e, 1);
  sorted_pair[row] = p;
  pair_row[p] = row;
}

// Tile = up to 64 sorted rows of one expert x 64 features; 256 threads, thread = 4 rows x 4 features; plain fp32 FMAs in k order.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TI* __restrict__ x, long long ldx, const int* __restrict__ sorted_pair, int src_div,
                                                       const TI* __restrict__ w, long long expert_stride, long long ldw, TO* __restrict__ out,
                                                       long long ldo, const int* __restrict__ plan, int F, int K, int act, long long x_off,
                                                       long long out_off) {
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[4 + 3 * tile], r0 = plan[4 + 3 * tile + 1], nr = plan[4 + 3 * tile + 2];
  const int f0 = blockIdx.x * 64;
  x += e * x_off;      // batched use: every "expert" reads its own column slice of x and writes its own slice of out
  out += e * out_off;
  __shared__ float xs[16][MOE_TILE + 4];
  __shared__ float ws[16][64 + 4];
  __shared__ long long src[MOE_TILE];
  if (threadIdx.x < MOE_TILE) {
    long long s = -1;
    if (threadIdx.x < nr) s = src_div > 0 ? sorted_pair[r0 + threadIdx.x] / src_div : (long long)(r0 + threadIdx.x);
    src[threadIdx.x] = s;
  }
  __syncthreads();
  const TI* we = w + (long long)e * expert_stride;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // features 4 tx .. + 4, rows 4 ty .. + 4
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < MOE_TILE * 16; i += 256) {
      const int r = i >> 4, k = i & 15;
      xs[k][r] = (src[r] >= 0 && k0 + k < K) ? ldm(x, src[r] * ldx + k0 + k) : 0.f;
    }
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, k = i & 15;
      ws[k][r] = (f0 + r < F && k0 + k < K) ? ldm(we, (long long)(f0 + r) * ldw + k0 + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  if (act == 3) {  // rows of w alternate gate / up: out[:, f / 2] = silu(gate) * up, both held by this thread
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int r = 4 * ty + i, f = f0 + tx * 4 + j;
        if (r < nr && f + 1 < F) {
          const float gv = acc[i][j];
          stm(out, (long long)(r0 + r) * ldo + f / 2, gv / (1.0f + expf(-gv)) * acc[i][j + 1]);
        }
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = 4 * ty + i, f = f0 + tx * 4 + j;
      if (r < nr && f < F) {
        float v = acc[i][j];
        if (act == 2) { v = fmaxf(v, 0.f); v *= v; }
        stm(out, (long long)(r0 + r) * ldo + f, v);
      }
    }
}

// The same product for bf16 operands on the tensor cores (mma.sync m16n8k16, fp32 accumulation): tile = 64 sorted rows of one
// expert x 128 (or 64) features, 4 warps of 32 x 64 (32), k in steps of 64 through a three-slot shared-memory ring filled by
// cp.async (16-byte pieces; the x rows are gathered through the sorted order), two steps in flight while one is multiplied.
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async_16(bf16* smem_dst, const bf16* gmem_src) {
  const uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(a), "l"(gmem_src) : "memory");
}

constexpr int MOE_KT = 64;           // k step of the tensor-core kernel
constexpr int MOE_LD = MOE_KT + 8;   // bf16 elements per shared row (conflict-free fragment reads)
constexpr int MOE_STAGES = 3;        // k steps in flight (cp.async ring)

template <typename TO, int BN>
__global__ void __launch_bounds__(128) moe_gemm_mma_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ sorted_pair, int src_div,
                                                           const bf16* __restrict__ w, long long expert_stride, long long ldw, TO* __restrict__ out,
                                                           long long ldo, const int* __restrict__ plan, int F, int K, int act, long long x_off,
                                                           long long out_off) {
  constexpr int KT = MOE_KT, LD = MOE_LD, ST = MOE_STAGES;
  constexpr int NI = BN / 16;  // 8-feature blocks per warp (two warps side by side)
  const int tile = blockIdx.y;
  if (tile >= plan[0]) return;
  const int e = plan[4 + 3 * tile], r0 = plan[4 + 3 * tile + 1], nr = plan[4 + 3 * tile + 2];
  const int f0 = blockIdx.x * BN;
  x += e * x_off;
  out += e * out_off;
  extern __shared__ __align__(16) unsigned char moe_smem[];
  bf16* As = reinterpret_cast<bf16*>(moe_smem);  // [ST][MOE_TILE][LD]
  bf16* Bs = As + ST * MOE_TILE * LD;            // [ST][BN][LD]
  __shared__ long long src[MOE_TILE];
  if (threadIdx.x < MOE_TILE) {
    long long s = -1;
    if (threadIdx.x < nr) s = src_div > 0 ? sorted_pair[r0 + threadIdx.x] / src_div : (long long)(r0 + threadIdx.x);
    src[threadIdx.x] = s;
  }
  __syncthreads();
  const bf16* we = w + (long long)e * expert_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gq = lane >> 2, tq = lane & 3;
  const int wm = warp >> 1, wn = warp & 1;
  // one k step of both operands into ring slot `stage`: 16-byte pieces, id -> row id / 8, columns 8 (id % 8); rows that do not
  // exist and columns past K are zeros
  auto issue = [&](int k0, int stage) {
    bf16* Ad = As + stage * MOE_TILE * LD;
    bf16* Bd = Bs + stage * BN * LD;
    for (int id = threadIdx.x; id < MOE_TILE * (KT / 8); id += 128) {
      const int r = id >> 3, c = (id & 7) * 8;
      bf16* d = Ad + r * LD + c;
      if (src[r] >= 0 && k0 + c < K) cp_async_16(d, x + src[r] * ldx + k0 + c);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    for (int id = threadIdx.x; id < BN * (KT / 8); id += 128) {
      const int r = id >> 3, c = (id & 7) * 8;
      bf16* d = Bd + r * LD + c;
      if (f0 + r < F && k0 + c < K) cp_async_16(d, we + (long long)(f0 + r) * ldw + k0 + c);
      else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
  };
  float acc[2][NI][4];
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni) acc[mi][ni][0] = acc[mi][ni][1] = acc[mi][ni][2] = acc[mi][ni][3] = 0.f;
  const int nk = (K + KT - 1) / KT;
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) {
    if (s < nk) issue(s * KT, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < nk; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(ST - 2) : "memory");  // k step kt has landed
    __syncthreads();                                                    // ... for every thread; slot (kt - 1) % ST is free again
    if (kt + ST - 1 < nk) issue((kt + ST - 1) * KT, (kt + ST - 1) % ST);
    asm volatile("cp.async.commit_group;" ::: "memory");
    const bf16* Ac = As + (kt % ST) * MOE_TILE * LD;
    const bf16* Bc = Bs + (kt % ST) * BN * LD;
#pragma unroll
    for (int ks = 0; ks < KT / 16; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const bf16* ap = Ac + (32 * wm + 16 * mi + gq) * LD + ks * 16 + 2 * tq;
        a[mi][0] = *reinterpret_cast<const uint32_t*>(ap);
        a[mi][1] = *reinterpret_cast<const uint32_t*>(ap + 8 * LD);
        a[mi][2] = *reinterpret_cast<const uint32_t*>(ap + 8);
        a[mi][3] = *reinterpret_cast<const uint32_t*>(ap + 8 * LD + 8);
      }
#pragma unroll
      for (int ni = 0; ni < NI; ++ni) {
        const bf16* bp = Bc + ((BN / 2) * wn + 8 * ni + gq) * LD + ks * 16 + 2 * tq;
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp), b1 = *reinterpret_cast<const uint32_t*>(bp + 8);
        mma_bf16_16816(acc[0][ni], a[0], b0, b1);
        mma_bf16_16816(acc[1][ni], a[1], b0, b1);
      }
    }
  }
  if (act == 3) {  // rows of w alternate gate / up: accumulator columns (2 tq, 2 tq + 1) are one output feature's pair
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int ni = 0; ni < NI; ++ni)
#pragma unroll
        for (int c = 0; c < 4; c += 2) {
          const int r = 32 * wm + 16 * mi + gq + ((c & 2) ? 8 : 0), f = f0 + (BN / 2) * wn + 8 * ni + 2 * tq;
          if (r < nr && f + 1 < F) {
            const float gv = acc[mi][ni][c];
            stm(out, (long long)(r0 + r) * ldo + f / 2, gv / (1.0f + expf(-gv)) * acc[mi][ni][c + 1]);
          }
        }
    return;
  }
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int ni = 0; ni < NI; ++ni)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = 32 * wm + 16 * mi + gq + ((c & 2) ? 8 : 0), f = f0 + (BN / 2) * wn + 8 * ni + 2 * tq + (c & 1);
        if (r < nr && f < F) {
          float v = acc[mi][ni][c];
          if (act == 2) { v = fmaxf(v, 0.f); v *= v; }
          stm(out, (long long)(r0 + r) * ldo + f, v);
        }
      }
}

template <typename TO, int BN>
static int launch_moe_mma(dim3 grid, cudaStream_t st, const void* x, long long ldx, const int* sorted_pair, int src_div, const void* w, long long expert_stride,
                          long long ldw, void* out, long long ldo, const int* plan, int F, int K, int act, long long x_off, long long out_off) {
  const size_t smem = (size_t)MOE_STAGES * (MOE_TILE + BN) * MOE_LD * sizeof(bf16);
  auto kern = moe_gemm_mma_kernel<TO, BN>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return PG_ERR_CUDA;
  kern<<<grid, 128, smem, st>>>(static_cast<const bf16*>(x), ldx, sorted_pair, src_div, static_cast<const bf16*>(w), expert_stride, ldw, static_cast<TO*>(out), ldo,
                                plan, F, K, act, x_off, out_off);
  pg_count_launch(1);
  return cudaGetLastError() == cudaSuccess ? PG_OK : PG_ERR_CUDA;
}

// xg[row, :] = x[sorted_pair[row] / top, :] for the `rows` sorted pairs that exist (rows read from offsets[n_real] on the device)
template <typename TA>
__global__ void moe_gather_rows_kernel(const TA* __restrict__ x, long long ldx, const int* __restrict__ sorted_pair, const int* __restrict__ total,
                                       int top, TA* __restrict__ xg, long long ldg, int D) {
  const int n = *total;
  for (int row = blockIdx.x; row < n; row += gridDim.x) {
    const TA* src = x + (long long)(sorted_pair[row] / top) * ldx;
    TA* dst = xg + (long long)row * ldg;
    for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
  }
}

template <typename TA>
__global__ void moe_combine_kernel(const float* __restrict__ expert_out, long long ldy, const int* __restrict__ pair_row, const int* __restrict__ ids,
                                   const float* __restrict__ weights, const TA* __restrict__ h, long long ldh, const float* __restrict__ shared_out,
                                   long long lds, float* __restrict__ y, int D, int top, const float* __restrict__ shared_gate, long long ldsg,
                                   int accumulate) {
  const long long t = blockIdx.x;
  const float sgate = shared_gate != nullptr ? 1.0f / (1.0f + expf(-shared_gate[t * ldsg])) : 1.0f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int row = pair_row[t * top + k];
      const float wgt = weights[t * top + k];
      const float v = row < 0 ? ldm(h, t * ldh + d) : expert_out[(long long)row * ldy + d];
      acc = fmaf(wgt, v, acc);
    }
    if (shared_out != nullptr) acc = fmaf(sgate, shared_out[t * lds + d], acc);
    y[t * D + d] = accumulate ? y[t * D + d] + acc : acc;
  }
}

}  // namespace

extern "C" int pg_moe_route(const float* logits, long long ld, const float* correction, int* ids, float* weights, int* counts, int tokens, int n_all,
                            int n_real, int top, int group_count, int group_keep, float scale, const float* logit_bias, void* stream) {
  if (tokens <= 0 || n_all <= 0 || n_real < 0 || n_real > n_all || top <= 0 || top > n_all) return PG_ERR_ARG;
  if (group_count > 1 && (n_all % group_count != 0 || group_keep <= 0 || group_keep > group_count || group_count > 256)) return PG_ERR_ARG;
  if (group_count > 1 && top > (long long)group_keep * (n_all / group_count)) return PG_ERR_ARG;
  const size_t smem = (size_t)4 * 2 * n_all * sizeof(float);
  if (smem > 48 * 1024) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  if (n_real > 0 && cudaMemsetAsync(counts, 0, (size_t)n_real * sizeof(int), st) != cudaSuccess) return PG_ERR_CUDA;
  moe_route_kernel<<<(tokens + 3) / 4, 128, smem, st>>>(logits, ld, correction, ids, weights, counts, tokens, n_all, n_real, top, group_count, group_keep,
                                                        scale, logit_bias);
  PG_RET();
}

extern "C" int pg_moe_tile_rows(void) { return MOE_TILE; }

extern "C" int pg_moe_plan(const int* counts, const int* ids, int* offsets, int* fill, int* plan, int* sorted_pair, int* pair_row, int pairs,
                           int n_real, int max_tiles, void* stream) {
  if (pairs <= 0 || n_real <= 0 || max_tiles <= 0) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  moe_plan_kernel<<<1, 32, 0, st>>>(counts, offsets, fill, plan, n_real, max_tiles);
  pg_count_launch(1);
  moe_scatter_kernel<<<(pairs + 255) / 256, 256, 0, st>>>(ids, offsets, fill, sorted_pair, pair_row, pairs, n_real);
  PG_RET();
}

extern "C" int pg_moe_gemm(const void* x, long long ldx, const int* sorted_pair, int src_div, const void* w, long long expert_stride, long long ldw,
                           void* out, long long ldo, const int* plan, int max_tiles, int F, int K, int act, int in_f32, int out_f32, long long x_expert_off,
                           long long out_expert_off, void* stream) {
  if (max_tiles <= 0 || max_tiles > 65535 || F <= 0 || K <= 0 || src_div < 0 || (act == 3 && (F & 1))) return PG_ERR_ARG;
  dim3 grid((F + 63) / 64, max_tiles);
  cudaStream_t st = PG_ST(stream);
  // bf16 operands whose rows can be fetched in 16-byte pieces go to the tensor cores
  if (!in_f32 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && expert_stride % 8 == 0 && x_expert_off % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) {
    // few tiles (decode: a handful of rows per expert, the weights stream once): narrower feature tiles for more CTAs in flight
    const bool narrow = (long long)max_tiles * ((F + 127) / 128) < 2LL * pg::num_sms();
    const int BN = narrow ? 64 : 128;
    dim3 g2((F + BN - 1) / BN, max_tiles);
#define PG_MOE_MMA(TO, BNV) \
  return launch_moe_mma<TO, BNV>(g2, st, x, ldx, sorted_pair, src_div, w, expert_stride, ldw, out, ldo, plan, F, K, act, x_expert_off, out_expert_off)
    if (out_f32) { if (narrow) PG_MOE_MMA(float, 64); else PG_MOE_MMA(float, 128); }
    else { if (narrow) PG_MOE_MMA(bf16, 64); else PG_MOE_MMA(bf16, 128); }
#undef PG_MOE_MMA
  }
  if (in_f32 && out_f32)
    moe_gemm_kernel<float, float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), ldx, sorted_pair, src_div, static_cast<const float*>(w), expert_stride,
                                                       ldw, static_cast<float*>(out), ldo, plan, F, K, act, x_expert_off, out_expert_off);
  else if (!in_f32 && out_f32)
    moe_gemm_kernel<bf16, float><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, sorted_pair, src_div, static_cast<const bf16*>(w), expert_stride,
                                                      ldw, static_cast<float*>(out), ldo, plan, F, K, act, x_expert_off, out_expert_off);
  else if (!in_f32 && !out_f32)
    moe_gemm_kernel<bf16, bf16><<<grid, 256, 0, st>>>(static_cast<const bf16*>(x), ldx, sorted_pair, src_div, static_cast<const bf16*>(w), expert_stride,
                                                     ldw, static_cast<bf16*>(out), ldo, plan, F, K, act, x_expert_off, out_expert_off);
  else
    return PG_ERR_ARG;
  PG_RET();
}

extern "C" int pg_moe_gather_rows(const void* x, long long ldx, const int* sorted_pair, const int* total_rows, int top, void* xg, long long ldg,
                                  int max_rows, int D, int act_f32, void* stream) {
  if (max_rows <= 0 || D <= 0 || top <= 0) return PG_ERR_ARG;
  const int grid = max_rows < 16384 ? max_rows : 16384;
  if (act_f32)
    moe_gather_rows_kernel<float><<<grid, 128, 0, PG_ST(stream)>>>(static_cast<const float*>(x), ldx, sorted_pair, total_rows, top, static_cast<float*>(xg), ldg, D);
  else
    moe_gather_rows_kernel<bf16><<<grid, 128, 0, PG_ST(stream)>>>(static_cast<const bf16*>(x), ldx, sorted_pair, total_rows, top, static_cast<bf16*>(xg), ldg, D);
  PG_RET();
}

// Every expert's run of gathered rows through two dense tensor-core products (tcgen05 kernels of pg_gemm_bf16), issued from
// here so that a layer costs one call from the host: mid = relu(xg W_up^T)^2 (bf16), eo = mid W_down^T (fp32).  One run is a few
// dozen output tiles -- a fraction of the SMs -- so the experts are spread over four side streams that fork from and join the
// caller's stream (the two products of one expert stay in order on one of them).
namespace {
constexpr int kSideStreams = 4;
struct SideStreams {
  cudaStream_t s[kSideStreams];
  cudaEvent_t fork, join[kSideStreams];
  bool ok = false;
};
SideStreams* side_streams() {
  static SideStreams per_device[16];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  SideStreams& ss = per_device[dev];
  if (!ss.ok) {
    if (cudaEventCreateWithFlags(&ss.fork, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    for (int i = 0; i < kSideStreams; ++i)
      if (cudaStreamCreateWithFlags(&ss.s[i], cudaStreamNonBlocking) != cudaSuccess ||
          cudaEventCreateWithFlags(&ss.join[i], cudaEventDisableTiming) != cudaSuccess)
        return nullptr;
    ss.ok = true;
  }
  return &ss;
}
}  // namespace

extern "C" int pg_moe_dense_runs(const void* xg, long long ldx, const void* w_up, const void* w_down, void* mid, long long ldm, float* eo, long long ldo,
                                 const int* counts_host, int n_real, int D, int F, int glu, void* stream) {
  if (n_real <= 0 || D <= 0 || F <= 0 || counts_host == nullptr || (glu && (F % 64) != 0)) return PG_ERR_ARG;
  const int up_rows = glu ? 2 * F : F;  // gated experts: [64 gate | 64 up] packed rows, the gated unit in the product's epilogue
  const bf16* x = static_cast<const bf16*>(xg);
  const bf16* wu = static_cast<const bf16*>(w_up);
  const bf16* wd = static_cast<const bf16*>(w_down);
  bf16* m = static_cast<bf16*>(mid);
  cudaStream_t main_st = PG_ST(stream);
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  SideStreams* ss = nullptr;
  if (cudaStreamIsCapturing(main_st, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) ss = side_streams();
  if (ss != nullptr) {
    if (cudaEventRecord(ss->fork, main_st) != cudaSuccess) return PG_ERR_CUDA;
    for (int i = 0; i < kSideStreams; ++i)
      if (cudaStreamWaitEvent(ss->s[i], ss->fork, 0) != cudaSuccess) return PG_ERR_CUDA;
  }
  long long off = 0;
  int rc = PG_OK, used = 0;
  for (int e = 0; e < n_real && rc == PG_OK; ++e) {
    const int c = counts_host[e];
    if (c <= 0) continue;
    void* st = ss != nullptr ? static_cast<void*>(ss->s[used++ % kSideStreams]) : stream;
    const int swap = c <= 128 ? 1 : 0;
    rc = pg_gemm_bf16(x + off * ldx, ldx, wu + (long long)e * up_rows * D, D, m + off * ldm, ldm, nullptr, nullptr, 0, c, up_rows, D,
                      glu ? PG_EPI_GEGLU : PG_EPI_BF16, glu ? 3 : 2, 1.0f, swap, 1, st);
    if (rc == PG_OK)
      rc = pg_gemm_bf16(m + off * ldm, ldm, wd + (long long)e * D * F, F, eo + off * ldo, ldo, nullptr, nullptr, 0, c, D, F, PG_EPI_F32, 0, 1.0f, swap, 1, st);
    off += c;
  }
  if (ss != nullptr)  // join even after an error: the caller's stream must not run ahead of work already issued
    for (int i = 0; i < kSideStreams; ++i)
      if (cudaEventRecord(ss->join[i], ss->s[i]) != cudaSuccess || cudaStreamWaitEvent(main_st, ss->join[i], 0) != cudaSuccess) return PG_ERR_CUDA;
  return rc;
}

extern "C" int pg_moe_combine(const float* expert_out, long long ldy, const int* pair_row, const int* ids, const float* weights, const void* h,
                              long long ldh, const float* shared_out, long long lds, float* y, int tokens, int D, int top, int act_f32,
                              const float* shared_gate, long long ldsg, int accumulate, void* stream) {
  if (tokens <= 0 || D <= 0 || top <= 0) return PG_ERR_ARG;
  cudaStream_t st = PG_ST(stream);
  if (act_f32)
    moe_combine_kernel<float><<<tokens, 256, 0, st>>>(expert_out, ldy, pair_row, ids, weights, static_cast<const float*>(h), ldh, shared_out, lds, y, D, top, shared_gate, ldsg, accumulate);
  else
    moe_combine_kernel<bf16><<<tokens, 256, 0, st>>>(expert_out, ldy, pair_row, ids, weights, static_cast<const bf16*>(h), ldh, shared_out, lds, y, D, top, shared_gate, ldsg, accumulate);
  PG_RET();
}
