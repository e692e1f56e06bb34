// A gated linear recurrence with a matrix state per head (the HGRN2 form): for head a of a request, with q, f in R^D and v in R^V,
//     S <- diag(f) S + (1 - f) v^T,    o = S^T q,      f = lower + (1 - lower) * sigmoid(z_f + b_f),   q = silu(z_q)
// where z_q, z_f, v are the rows [q | f | v] of one fused projection (float32 partial sums, added in order). The state S [D, V] is
// float32, lives in the request's state slot, starts at zero and is carried from token to token; everything here is float32.
//
//  * gated_recurrence: one CTA per (segment, head, 32 or 16 value columns). A thread owns one column j and every DS-th row of S in registers;
//    the tokens of the segment are walked in order, sixteen at a time: the CTA first turns the sixteen tokens' projections into q, f
//    and 1 - f in shared memory, then every thread updates its rows and adds its share of o[j], which a shuffle sums over the DS
//    threads of the column. A decoded token is a segment of one: the cost is then the state's trip from memory and back.
//  * head_rmsnorm: out[t, a, :] = w * o[t, a, :] / sqrt(mean(o^2) + eps), into the activation dtype.
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kChunk = 16;   // tokens prepared at a time

// RPT: rows of S a thread holds; kCols: value columns per CTA (32, or 16 where a thread holds sixteen rows: the CTA then has 512 threads at most)
template <int RPT, int kCols>
__global__ void __launch_bounds__(kCols * 32) gated_recurrence_kernel(const float* __restrict__ proj, int P, size_t stride_p, int R, const float* __restrict__ f_bias,
                                        const float* __restrict__ lower, float* __restrict__ state, size_t slot_stride, const int* __restrict__ seg_start,
                                        const int* __restrict__ seg_slot, float* __restrict__ o_out, int heads, int D, int V, int DS) {
  extern __shared__ float sm[];   // q[kChunk][D], f[kChunk][D], g[kChunk][D], v[kChunk][kCols]
  float* sq = sm;
  float* sf = sq + kChunk * D;
  float* sg = sf + kChunk * D;
  float* sv = sg + kChunk * D;
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int s = blockIdx.x, a = blockIdx.y, j0 = blockIdx.z * kCols;
  const int tid = threadIdx.x, ds = tid % DS, col = tid / DS, j = j0 + col;
  const int t0 = seg_start[s], t1 = seg_start[s + 1];
  float* S = state + (size_t)seg_slot[s] * slot_stride + (size_t)a * D * V;
  float st[RPT];
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    const int d = ds + r * DS;
    st[r] = (d < D && j < V) ? S[(size_t)d * V + j] : 0.f;
  }
  const int q_off = a * D, f_off = heads * D + a * D, v_off = 2 * heads * D + a * V + j0;
  for (int c0 = t0; c0 < t1; c0 += kChunk) {
    const int n = min(kChunk, t1 - c0);
    __syncthreads();
    for (int i = tid; i < n * D; i += blockDim.x) {
      const int tt = i / D, d = i % D;
      const float* src = proj + (size_t)(c0 + tt) * R;
      float zq = src[q_off + d], zf = src[f_off + d];
      for (int p = 1; p < P; p++) zq += src[p * stride_p + q_off + d], zf += src[p * stride_p + f_off + d];
      zf += f_bias[a * D + d];
      const float lo = lower[a * D + d];
      const float sig = 1.f / (1.f + expf(-zf));
      const float f = __fmaf_rn(1.f - lo, sig, lo);
      sq[i] = zq / (1.f + expf(-zq));
      sf[i] = f;
      sg[i] = 1.f - f;
    }
    for (int i = tid; i < n * kCols; i += blockDim.x) {
      const int tt = i / kCols, c = i % kCols;
      float z = 0.f;
      if (j0 + c < V) {
        const float* src = proj + (size_t)(c0 + tt) * R + v_off + c;
        z = src[0];
        for (int p = 1; p < P; p++) z += src[p * stride_p];
      }
      sv[i] = z;
    }
    __syncthreads();
    for (int tt = 0; tt < n; tt++) {
      const float vj = sv[tt * kCols + col];
      const float* fq = sq + tt * D;
      const float* ff = sf + tt * D;
      const float* fg = sg + tt * D;
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < RPT; r++) {
        const int d = ds + r * DS;
        if (d < D) {
          st[r] = __fmaf_rn(ff[d], st[r], fg[d] * vj);
          acc = __fmaf_rn(st[r], fq[d], acc);
        }
      }
      for (int o = DS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (ds == 0 && j < V) o_out[((size_t)(c0 + tt) * heads + a) * V + j] = acc;
    }
  }
#pragma unroll
  for (int r = 0; r < RPT; r++) {
    const int d = ds + r * DS;
    if (d < D && j < V) S[(size_t)d * V + j] = st[r];
  }
}

template <typename O>
__global__ void head_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps, O* __restrict__ out, long long items, int V) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= items) return;
  const float* src = o + item * V;
  float ss = 0.f;
  for (int i = lane; i < V; i += 32) ss = __fmaf_rn(src[i], src[i], ss);
  const float inv = rsqrtf(ib::warp_sum(ss) / (float)V + eps);
  for (int i = lane; i < V; i += 32) out[item * V + i] = ib::from_f32<O>(w[i] * (src[i] * inv));
}

}  // namespace

extern "C" int ib_gated_recurrence(const float* proj, int P, long long stride_p, const float* f_bias, const float* lower, float* state, long long slot_stride,
                                   const int* seg_start, const int* seg_slot, int n_segments, float* o_out, int heads, int D, int V, cudaStream_t stream) {
  if (n_segments == 0) return 0;
  IB_CHECK_ARG(n_segments > 0 && P >= 1 && heads > 0 && D > 0 && V > 0, "gated_recurrence: bad sizes segments=%d P=%d heads=%d D=%d V=%d", n_segments, P, heads, D, V);
  IB_CHECK_ARG(D <= 512, "gated_recurrence: a head's key size %d is above 512", D);
  const int rpt = D <= 256 ? 8 : 16, kCols = D <= 256 ? 32 : 16;
  IB_CHECK_ARG(heads <= 65535 && (V + kCols - 1) / kCols <= 65535, "gated_recurrence: the grid is too large");
  int DS = 1;
  while (DS * rpt < D) DS *= 2;
  const int R = 2 * heads * D + heads * V;
  const size_t smem = (size_t)kChunk * (3 * D + kCols) * sizeof(float);
  const dim3 grid((unsigned)n_segments, (unsigned)heads, (unsigned)((V + kCols - 1) / kCols));
  auto go = [&](auto kernel) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kCols * DS, smem, stream, proj, P, (size_t)stride_p, R, f_bias, lower, state, (size_t)slot_stride, seg_start, seg_slot, o_out, heads, D, V, DS);
  };
  if (rpt == 8) go(gated_recurrence_kernel<8, 32>);
  else go(gated_recurrence_kernel<16, 16>);
  IB_CHECK_LAUNCH("gated_recurrence");
  return 0;
}

extern "C" int ib_head_rmsnorm(const float* o, const float* w, float eps, void* out, int out_dtype, long long items, int V, cudaStream_t stream) {
  if (items == 0) return 0;
  IB_CHECK_ARG(items > 0 && V > 0, "head_rmsnorm: bad sizes items=%lld V=%d", items, V);
  const unsigned grid = (unsigned)((items + 3) / 4);
  if (out_dtype == IB_F32) ib::launch(head_rmsnorm_kernel<float>, grid, 128, 0, stream, o, w, eps, (float*)out, items, V);
  else if (out_dtype == IB_BF16) ib::launch(head_rmsnorm_kernel<__nv_bfloat16>, grid, 128, 0, stream, o, w, eps, (__nv_bfloat16*)out, items, V);
  else return ib_set_error("head_rmsnorm: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("head_rmsnorm");
  return 0;
}
