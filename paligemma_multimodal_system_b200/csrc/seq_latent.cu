// Latent attention (keys and values of every head are linear images of one low-rank row per token, plus one rotated key part
// shared by the heads): what the cache keeps per token is  [c (rank) | r (rot)]  -- the normalised latent and the rotated part.
//
//   pg_latent_prepare   from the joint down projection [q latent | kv latent | rotated key part | ...] of a row: RMS norm of
//                       the q latent (-> dense buffer, operand of the q up projection), RMS norm of the kv latent and the
//                       pairwise rotation of the key part (-> the token's row in the cache pages)
//   pg_rotate_heads     pairwise rotation of a slice of every head vector by the row's position, written to another layout
//                       (q's rotated part into the absorbed query, or q / k as a whole)
//   pg_latent_gather    explicit-head form, step 1: the latent rows of every multi-token entry's context + new tokens are gathered
//                       into a dense matrix (entry e from row dense_row0[e]), the operand of the key / value up projection
//   pg_latent_pack_kv   [k_plain heads | v heads] of the up projection + the shared rotated part -> per-head key rows
//                       [plain | rotated] and value rows in dense scratch "pages"
//
// Norm statistics and angles are fp32 / double; the stored rows have the activation type.
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

template <typename T>
__device__ __forceinline__ float ldv(const T* p, long long i);
template <>
__device__ __forceinline__ float ldv<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ldv<bf16>(const bf16* p, long long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stv(float* p, long long i, float v) { p[i] = v; }
__device__ __forceinline__ void stv(bf16* p, long long i, float v) { p[i] = __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum128(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3];
}

// One CTA (128 threads) per token row.
template <typename TA>
__global__ void __launch_bounds__(128) latent_prepare_kernel(const TA* __restrict__ proj, long long ld, const int* __restrict__ pos,
                                                             const int* __restrict__ row_entry, const int* __restrict__ page_table, int max_pages,
                                                             int page, const double* __restrict__ freq, const float* __restrict__ qn,
                                                             const float* __restrict__ cn, TA* __restrict__ cq_out, TA* __restrict__ pages,
                                                             int q_rank, int rank, int rot, int rot_dims, float eps, float rot_gain) {
  __shared__ float red[4];
  const long long t = blockIdx.x;
  const TA* row = proj + t * ld;
  const int p = pos[t];
  if (q_rank > 0) {
    float s = 0.f;
    for (int d = threadIdx.x; d < q_rank; d += 128) { const float v = ldv(row, d); s = fmaf(v, v, s); }
    s = block_sum128(s, red);
    const float inv = 1.0f / sqrtf(s / (float)q_rank + eps);
    for (int d = threadIdx.x; d < q_rank; d += 128) stv(cq_out, t * q_rank + d, ldv(row, d) * inv * qn[d]);
  }
  if (pages == nullptr) return;  // a layer that attends over another layer's cached rows prepares its query latent only
  const long long pg_row = (long long)page_table[(long long)row_entry[t] * max_pages + p / page] * page + p % page;
  TA* dst = pages + pg_row * (long long)(rank + rot);
  {
    float s = 0.f;
    for (int d = threadIdx.x; d < rank; d += 128) { const float v = ldv(row, q_rank + d); s = fmaf(v, v, s); }
    s = block_sum128(s, red);
    const float inv = 1.0f / sqrtf(s / (float)rank + eps);
    for (int d = threadIdx.x; d < rank; d += 128) stv(dst, d, ldv(row, q_rank + d) * inv * cn[d]);
  }
  const TA* r = row + q_rank + rank;
  for (int i = threadIdx.x; 2 * i < rot; i += 128) {
    const int d = 2 * i;
    float a = ldv(r, d), b = d + 1 < rot ? ldv(r, d + 1) : 0.f;
    if (d + 1 < rot_dims) {
      double sn, c;
      sincos((double)p * freq[i], &sn, &c);
      const float cf = (float)c * rot_gain, sf = (float)sn * rot_gain;
      const float ra = a * cf - b * sf, rb = b * cf + a * sf;
      a = ra; b = rb;
    }
    stv(dst, rank + d, a);
    if (d + 1 < rot) stv(dst, rank + d + 1, b);
  }
}

// grid (rows, head blocks); thread <-> (head, pair)
template <typename TA>
__global__ void rotate_heads_kernel(const TA* __restrict__ src, long long ld_src, long long hs_src, TA* __restrict__ dst, long long ld_dst,
                                    long long hs_dst, const int* __restrict__ pos, const double* __restrict__ freq, int H, int n, int rot_dims,
                                    float rot_gain) {
  extern __shared__ float cs[];  // cos, sin of the row's rot_dims/2 angles
  const long long t = blockIdx.x;
  const int p = pos[t];
  for (int i = threadIdx.x; i < rot_dims / 2; i += blockDim.x) {
    double sn, c;
    sincos((double)p * freq[i], &sn, &c);
    cs[i] = (float)c * rot_gain;
    cs[rot_dims / 2 + i] = (float)sn * rot_gain;
  }
  __syncthreads();
  const int pairs = (n + 1) / 2;
  for (int idx = threadIdx.x; idx < H * pairs; idx += blockDim.x) {
    const int h = idx / pairs, d = 2 * (idx % pairs);
    const TA* s = src + t * ld_src + (long long)h * hs_src;
    TA* o = dst + t * ld_dst + (long long)h * hs_dst;
    float a = ldv(s, d), b = d + 1 < n ? ldv(s, d + 1) : 0.f;
    if (d + 1 < rot_dims) {
      const float c = cs[d >> 1], sn = cs[rot_dims / 2 + (d >> 1)];
      const float ra = a * c - b * sn, rb = b * c + a * sn;
      a = ra; b = rb;
    }
    stv(o, d, a);
    if (d + 1 < n) stv(o, d + 1, b);
  }
}

// dense row r of entry e (r < ctx + n) <- cached latent row of position r: the first `rank` columns to lat [rows, rank]
template <typename TA>
__global__ void latent_gather_kernel(const TA* __restrict__ pages, const int* __restrict__ page_table, int max_pages, int page,
                                     const int* __restrict__ dense_row0, const int* __restrict__ entry_n, const int* __restrict__ entry_ctx,
                                     TA* __restrict__ lat, int rank, int width) {
  const int e = blockIdx.y;
  if (entry_n[e] == 1) return;  // single-token entries are served by the absorbed form: they own no dense rows
  const int len = entry_ctx[e] + entry_n[e];
  for (int j = blockIdx.x; j < len; j += gridDim.x) {
    const TA* src = pages + ((long long)page_table[(long long)e * max_pages + j / page] * page + j % page) * width;
    TA* dst = lat + (long long)(dense_row0[e] + j) * rank;
    for (int d = threadIdx.x; d < rank; d += blockDim.x) dst[d] = src[d];
  }
}

// per dense row: k[row, h, :] = [up[row, h * dim ..] | rotated part of the cached row], v[row, h, :] = up[row, H * dim + h * vdim ..]
template <typename TA>
__global__ void latent_pack_kv_kernel(const TA* __restrict__ up, long long ld_up, const TA* __restrict__ pages, const int* __restrict__ page_table,
                                      int max_pages, int page, const int* __restrict__ dense_row0, const int* __restrict__ entry_n,
                                      const int* __restrict__ entry_ctx, TA* __restrict__ k_out, TA* __restrict__ v_out, int H, int dim, int rot,
                                      int vdim, int rank) {
  const int e = blockIdx.y;
  if (entry_n[e] == 1) return;
  const int len = entry_ctx[e] + entry_n[e];
  const int kd = dim + rot;
  for (int j = blockIdx.x; j < len; j += gridDim.x) {
    const long long row = dense_row0[e] + j;
    const TA* src = pages + ((long long)page_table[(long long)e * max_pages + j / page] * page + j % page) * (long long)(rank + rot) + rank;
    const TA* u = up + row * ld_up;
    TA* ko = k_out + row * (long long)H * kd;
    TA* vo = v_out + row * (long long)H * vdim;
    for (int i = threadIdx.x; i < H * kd; i += blockDim.x) {
      const int h = i / kd, d = i % kd;
      ko[i] = d < dim ? u[(long long)h * dim + d] : src[d - dim];
    }
    for (int i = threadIdx.x; i < H * vdim; i += blockDim.x) vo[i] = u[(long long)H * dim + i];
  }
}

}  // namespace

extern "C" int pg_latent_prepare(const void* proj, long long ld, const int* pos, const int* row_entry, const int* page_table, int max_pages,
                                 int page, const double* freq, const float* q_norm, const float* c_norm, void* cq_out, void* pages, int rows,
                                 int q_rank, int rank, int rot, int rot_dims, float eps, float rot_gain, int act_f32, void* stream) {
  if (rows <= 0 || q_rank < 0 || rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1) || page <= 0) return PG_ERR_ARG;
  if (pages == nullptr && q_rank == 0) return PG_ERR_ARG;
  if (act_f32)
    latent_prepare_kernel<float><<<rows, 128, 0, PG_ST(stream)>>>(static_cast<const float*>(proj), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                 q_norm, c_norm, static_cast<float*>(cq_out), static_cast<float*>(pages), q_rank, rank,
                                                                 rot, rot_dims, eps, rot_gain);
  else
    latent_prepare_kernel<bf16><<<rows, 128, 0, PG_ST(stream)>>>(static_cast<const bf16*>(proj), ld, pos, row_entry, page_table, max_pages, page, freq,
                                                                q_norm, c_norm, static_cast<bf16*>(cq_out), static_cast<bf16*>(pages), q_rank, rank,
                                                                rot, rot_dims, eps, rot_gain);
  PG_RET();
}

extern "C" int pg_rotate_heads(const void* src, long long ld_src, long long head_stride_src, void* dst, long long ld_dst, long long head_stride_dst,
                               const int* pos, const double* freq, int rows, int H, int n, int rot_dims, float rot_gain, int act_f32, void* stream) {
  if (rows <= 0 || H <= 0 || n <= 0 || rot_dims < 0 || rot_dims > n || (rot_dims & 1)) return PG_ERR_ARG;
  const size_t smem = (size_t)(rot_dims + 2) * sizeof(float);
  if (act_f32)
    rotate_heads_kernel<float><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const float*>(src), ld_src, head_stride_src, static_cast<float*>(dst),
                                                                  ld_dst, head_stride_dst, pos, freq, H, n, rot_dims, rot_gain);
  else
    rotate_heads_kernel<bf16><<<rows, 128, smem, PG_ST(stream)>>>(static_cast<const bf16*>(src), ld_src, head_stride_src, static_cast<bf16*>(dst), ld_dst,
                                                                 head_stride_dst, pos, freq, H, n, rot_dims, rot_gain);
  PG_RET();
}

extern "C" int pg_latent_gather(const void* pages, const int* page_table, int max_pages, int page, const int* dense_row0, const int* entry_n,
                                const int* entry_ctx, void* lat, int entries, int max_len, int rank, int width, int act_f32, void* stream) {
  if (entries <= 0 || entries > 65535 || max_len <= 0 || rank <= 0 || width < rank || page <= 0) return PG_ERR_ARG;
  dim3 grid(max_len < 4096 ? max_len : 4096, entries);
  if (act_f32)
    latent_gather_kernel<float><<<grid, 128, 0, PG_ST(stream)>>>(static_cast<const float*>(pages), page_table, max_pages, page, dense_row0, entry_n,
                                                                entry_ctx, static_cast<float*>(lat), rank, width);
  else
    latent_gather_kernel<bf16><<<grid, 128, 0, PG_ST(stream)>>>(static_cast<const bf16*>(pages), page_table, max_pages, page, dense_row0, entry_n,
                                                               entry_ctx, static_cast<bf16*>(lat), rank, width);
  PG_RET();
}

extern "C" int pg_latent_pack_kv(const void* up, long long ld_up, const void* pages, const int* page_table, int max_pages, int page,
                                 const int* dense_row0, const int* entry_n, const int* entry_ctx, void* k_out, void* v_out, int entries, int max_len,
                                 int H, int dim, int rot, int vdim, int rank, int act_f32, void* stream) {
  if (entries <= 0 || entries > 65535 || max_len <= 0 || H <= 0 || dim <= 0 || rot < 0 || vdim <= 0 || rank <= 0 || page <= 0) return PG_ERR_ARG;
  dim3 grid(max_len < 4096 ? max_len : 4096, entries);
  if (act_f32)
    latent_pack_kv_kernel<float><<<grid, 256, 0, PG_ST(stream)>>>(static_cast<const float*>(up), ld_up, static_cast<const float*>(pages), page_table,
                                                                 max_pages, page, dense_row0, entry_n, entry_ctx, static_cast<float*>(k_out),
                                                                 static_cast<float*>(v_out), H, dim, rot, vdim, rank);
  else
    latent_pack_kv_kernel<bf16><<<grid, 256, 0, PG_ST(stream)>>>(static_cast<const bf16*>(up), ld_up, static_cast<const bf16*>(pages), page_table,
                                                                max_pages, page, dense_row0, entry_n, entry_ctx, static_cast<bf16*>(k_out),
                                                                static_cast<bf16*>(v_out), H, dim, rot, vdim, rank);
  PG_RET();
}
