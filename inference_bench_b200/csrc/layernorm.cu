// Layer norm without a bias, fused with the residual add that precedes it, and the pieces of a block whose sublayers read
// their input through a short causal convolution over time and whose layers are mixed by a depth-weighted average.
// All arithmetic is float32; only a stored activation may be bfloat16.
//
//  * add_layernorm: v = x[t] + scale * (sum_p delta[p][t] + bias)   (scale, bias: per channel, optional; partial sums added in order)
//                   x[t] = v (optional), x_copy[t] = v (optional)
//                   out = w * (v - mean(v)) / sqrt(mean((v - mean)^2) + eps)
//    With `halo` > 0 the output rows are laid out for the convolution that follows: segment s (tokens a..b of the flat batch) owns
//    rows a + s * halo .. b + (s + 1) * halo; its first `halo` rows are the request's last `halo` normed rows of earlier steps, copied
//    from its state slot by extra blocks of this kernel, so the convolution reads one array and its state update races with nothing.
//  * causal_conv_rows: out[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j] on that layout, and the request's new state (the last
//    `halo` = taps - 1 rows of its extended run) written back to its slot.
//  * depth_average: X = x[t] + scale * (sum_p delta[p][t] + bias); stack[k][t] = X; x[t] = sum_{j <= k} mix[j] * stack[j][t].
//  * scale_values: v *= s (logits times a constant).
#include <type_traits>

#include "common.cuh"

namespace {

constexpr int kLnThreads = 256;

template <typename O>
__global__ void __launch_bounds__(kLnThreads) add_layernorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride,
                                                                   const float* __restrict__ dscale, const float* __restrict__ dbias,
                                                                   const float* __restrict__ w, O* __restrict__ out, const int* __restrict__ rows, int n_rows,
                                                                   int H, float eps, int write_x, float* __restrict__ x_copy, int halo,
                                                                   const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                                                   const int* __restrict__ seg_slot, const float* __restrict__ state, size_t slot_stride) {
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  const int r = blockIdx.x;
  if (r >= n_rows) {   // a halo row: the request's state of earlier steps, as it is
    const int hb = r - n_rows, s = hb / halo, j = hb % halo;
    const float* src = state + (size_t)seg_slot[s] * slot_stride + (size_t)j * H;
    O* dst = out + ((size_t)seg_start[s] + (size_t)s * halo + j) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ib::from_f32<O>(src[i]);
    return;
  }
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * H;
  float sum = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = xr[i];
    if (P > 0 || dbias) {
      float d = dbias ? dbias[i] : 0.f;
      if (P > 0) {
        float a = delta[(size_t)t * H + i];
        for (int p = 1; p < P; p++) a += delta[p * delta_stride + (size_t)t * H + i];
        d = dbias ? a + d : a;
      }
      v = dscale ? __fmaf_rn(dscale[i], d, v) : v + d;
      if (write_x) xr[i] = v;
    }
    if (x_copy) x_copy[(size_t)t * H + i] = v;
    row[i] = v;
    sum += v;
  }
  const float mean = ib::block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float c = row[i] - mean;
    sq = __fmaf_rn(c, c, sq);
  }
  const float inv = rsqrtf(ib::block_sum(sq, scratch) / (float)H + eps);
  const size_t orow = halo ? (size_t)t + (size_t)(seg_of_token[t] + 1) * halo : (size_t)r;
  O* dst = out + orow * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = ib::from_f32<O>((row[i] - mean) * inv * w[i]);
}

template <typename O>
__global__ void __launch_bounds__(kLnThreads) causal_conv_rows_kernel(const float* __restrict__ ext, const float* __restrict__ w, int taps, O* __restrict__ out,
                                                                      int T, int H, const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                                                      const int* __restrict__ seg_slot, float* __restrict__ state, size_t slot_stride) {
  // This kernel does not let its dependents start early. What follows it is a sublayer's first matrix product, which takes its tensor
  // memory before it waits; the product two kernels back (a mixer's output projection) may itself still be waiting for tensor memory
  // that an attention kernel holds, and a later, smaller request must not be served before it: the later kernel would then hold what
  // the earlier one needs while waiting for it. With no early start here, nothing after this kernel runs before the products before it
  // are done.
  ib::pdl_wait();
  const int halo = taps - 1;
  const int b = blockIdx.x;
  if (b >= T) {   // a halo row of segment s: it stays in the state when the step brought fewer than `halo` tokens
    const int hb = b - T, s = hb / halo, j = hb % halo;
    const int a = seg_start[s], n = seg_start[s + 1] - a;
    if (j < n) return;
    const float* src = ext + ((size_t)a + (size_t)s * halo + j) * H;
    float* dst = state + (size_t)seg_slot[s] * slot_stride + (size_t)(j - n) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    return;
  }
  const int t = b, s = seg_of_token[t];
  const int end = seg_start[s + 1];
  const float* cur = ext + ((size_t)t + (size_t)(s + 1) * halo) * H;
  float* keep = end - t <= halo ? state + (size_t)seg_slot[s] * slot_stride + (size_t)(halo - (end - t)) * H : nullptr;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float y = 0.f;
    for (int j = 0; j < taps; j++) y = __fmaf_rn(w[(size_t)i * taps + j], cur[(ptrdiff_t)(j - halo) * H + i], y);
    const float h = cur[i];
    out[(size_t)t * H + i] = ib::from_f32<O>(h + y);
    if (keep) keep[i] = h;
  }
}

__global__ void depth_average_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride, const float* __restrict__ dscale,
                                     const float* __restrict__ dbias, float* __restrict__ stack, size_t layer_stride, int k, const float* __restrict__ mix, int H) {
  // (no early start of the dependents, for the reason given in causal_conv_rows_kernel: in a layer without a feed-forward this kernel
  // is what stands between a mixer's output projection and the next matrix product)
  ib::pdl_wait();
  const size_t t = blockIdx.y;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) {
    const size_t at = t * H + i;
    float v = x[at];
    if (P > 0) {
      float a = delta[at];
      for (int p = 1; p < P; p++) a += delta[p * delta_stride + at];
      if (dbias) a += dbias[i];
      v = dscale ? __fmaf_rn(dscale[i], a, v) : v + a;
    }
    stack[(size_t)k * layer_stride + at] = v;
    float m = 0.f;
    for (int j = 0; j < k; j++) m = __fmaf_rn(mix[j], stack[(size_t)j * layer_stride + at], m);
    x[at] = __fmaf_rn(mix[k], v, m);
  }
}

__global__ void scale_values_kernel(float* __restrict__ v, size_t n, float s) {
  ib::pdl_launch_dependents();
  ib::pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) v[i] *= s;
}

}  // namespace

extern "C" int ib_add_layernorm(float* x, const float* delta, int P, long long delta_stride, const float* dscale, const float* dbias, const float* w, void* out,
                                int out_dtype, const int* rows, int n_rows, int H, float eps, int write_x, float* x_copy, int halo, const int* seg_of_token,
                                const int* seg_start, const int* seg_slot, int n_segments, const float* state, long long slot_stride, cudaStream_t stream) {
  if (n_rows == 0) return 0;
  IB_CHECK_ARG(n_rows > 0 && H > 0 && P >= 0 && halo >= 0, "add_layernorm: bad sizes rows=%d H=%d P=%d halo=%d", n_rows, H, P, halo);
  IB_CHECK_ARG(!(halo && rows), "add_layernorm: gathered rows have no layout for a convolution");
  IB_CHECK_ARG(!halo || (seg_of_token && seg_start && seg_slot && state && n_segments > 0), "add_layernorm: the convolution's layout needs the step's segments and the state");
  const size_t smem = (size_t)H * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "add_layernorm: rows of %d values do not fit in shared memory", H);
  const unsigned grid = (unsigned)n_rows + (unsigned)(halo * (halo ? n_segments : 0));
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, grid, kLnThreads, smem, stream, x, delta, P, (size_t)delta_stride, dscale, dbias, w, o, rows, n_rows, H, eps, write_x, x_copy, halo, seg_of_token,
               seg_start, seg_slot, state, (size_t)slot_stride);
  };
  if (out_dtype == IB_F32) go(add_layernorm_kernel<float>, (float*)out);
  else if (out_dtype == IB_BF16) go(add_layernorm_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
  else return ib_set_error("add_layernorm: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("add_layernorm");
  return 0;
}

extern "C" int ib_causal_conv_rows(const float* ext, const float* w, int taps, void* out, int out_dtype, int T, int H, const int* seg_of_token, const int* seg_start,
                                   const int* seg_slot, int n_segments, float* state, long long slot_stride, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && taps >= 1 && n_segments > 0, "causal_conv_rows: bad sizes T=%d H=%d taps=%d segments=%d", T, H, taps, n_segments);
  const unsigned grid = (unsigned)T + (unsigned)((taps - 1) * n_segments);
  if (out_dtype == IB_F32)
    ib::launch(causal_conv_rows_kernel<float>, grid, kLnThreads, 0, stream, ext, w, taps, (float*)out, T, H, seg_of_token, seg_start, seg_slot, state, (size_t)slot_stride);
  else if (out_dtype == IB_BF16)
    ib::launch(causal_conv_rows_kernel<__nv_bfloat16>, grid, kLnThreads, 0, stream, ext, w, taps, (__nv_bfloat16*)out, T, H, seg_of_token, seg_start, seg_slot, state,
               (size_t)slot_stride);
  else return ib_set_error("causal_conv_rows: unknown output dtype %d", out_dtype);
  IB_CHECK_LAUNCH("causal_conv_rows");
  return 0;
}

extern "C" int ib_depth_average(float* x, const float* delta, int P, long long delta_stride, const float* dscale, const float* dbias, float* stack, long long layer_stride, int k,
                                const float* mix, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && k >= 1 && P >= 0, "depth_average: bad sizes T=%d H=%d k=%d P=%d", T, H, k, P);
  IB_CHECK_ARG(T <= 65535, "depth_average: T=%d rows exceed the grid limit 65535", T);
  ib::launch(depth_average_kernel, dim3(min((H + 255) / 256, 32), T), 256, 0, stream, x, delta, P, (size_t)delta_stride, dscale, dbias, stack, (size_t)layer_stride, k, mix, H);
  IB_CHECK_LAUNCH("depth_average");
  return 0;
}

extern "C" int ib_scale_values(float* v, long long n, float s, cudaStream_t stream) {
  if (n <= 0) return 0;
  ib::launch(scale_values_kernel, (unsigned)min((long long)1024, (n + 255) / 256), 256, 0, stream, v, (size_t)n, s);
  IB_CHECK_LAUNCH("scale_values");
  return 0;
}
