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
//  * causal_conv_rows: out[t] = h[t] + sum_j w[j, :] * h[t - taps + 1 + j] on that layout (w is [taps][channels]: a tap's weights lie together), and the request's new state (the last
//    `halo` = taps - 1 rows of its extended run) written back to its slot.
//  * add_layernorm_conv_single: both of the above in one kernel for a step in which every request brings one token (decoded tokens): a CTA
//    per token norms its row, reads the request's `halo` state rows, writes the convolved row and shifts the state by one row.
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
    for (int j = 0; j < taps; j++) y = __fmaf_rn(w[(size_t)j * H + i], cur[(ptrdiff_t)(j - halo) * H + i], y);
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

// ---- the same three kernels with 16-byte accesses, for rows of a multiple of four values (every sum runs in the order of the scalar forms)
__device__ __forceinline__ float4 ld4(const float* p) { return *(const float4*)p; }
__device__ __forceinline__ void st4(float* p, float4 v) { *(float4*)p = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  *(uint2*)p = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
}
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
__device__ __forceinline__ float4 fma4(float4 a, float4 b, float4 c) {
  return make_float4(__fmaf_rn(a.x, b.x, c.x), __fmaf_rn(a.y, b.y, c.y), __fmaf_rn(a.z, b.z, c.z), __fmaf_rn(a.w, b.w, c.w));
}

template <typename O>
__global__ void __launch_bounds__(kLnThreads) add_layernorm_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride,
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
  if (r >= n_rows) {
    const int hb = r - n_rows, s = hb / halo, j = hb % halo;
    const float* src = state + (size_t)seg_slot[s] * slot_stride + (size_t)j * H;
    O* dst = out + ((size_t)seg_start[s] + (size_t)s * halo + j) * H;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) st4(dst + i, ld4(src + i));
    return;
  }
  const int t = rows ? rows[r] : r;
  float* xr = x + (size_t)t * H;
  float sum = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = ld4(xr + i);
    if (P > 0 || dbias) {
      float4 d = dbias ? ld4(dbias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (P > 0) {
        float4 a = ld4(delta + (size_t)t * H + i);
        for (int p = 1; p < P; p++) a = add4(a, ld4(delta + p * delta_stride + (size_t)t * H + i));
        d = dbias ? add4(a, d) : a;
      }
      v = dscale ? fma4(ld4(dscale + i), d, v) : add4(v, d);
      if (write_x) st4(xr + i, v);
    }
    if (x_copy) st4(x_copy + (size_t)t * H + i, v);
    st4(row + i, v);
    sum += (v.x + v.y) + (v.z + v.w);
  }
  const float mean = ib::block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = ld4(row + i);
    const float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
    sq = __fmaf_rn(e, e, __fmaf_rn(c, c, __fmaf_rn(b, b, __fmaf_rn(a, a, sq))));
  }
  const float inv = rsqrtf(ib::block_sum(sq, scratch) / (float)H + eps);
  const size_t orow = halo ? (size_t)t + (size_t)(seg_of_token[t] + 1) * halo : (size_t)r;
  O* dst = out + orow * H;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = ld4(row + i), g = ld4(w + i);
    st4(dst + i, make_float4((v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y, (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w));
  }
}

template <typename O>
__global__ void __launch_bounds__(kLnThreads) causal_conv_rows_vec_kernel(const float* __restrict__ ext, const float* __restrict__ w, int taps, O* __restrict__ out,
                                                                          int T, int H, const int* __restrict__ seg_of_token, const int* __restrict__ seg_start,
                                                                          const int* __restrict__ seg_slot, float* __restrict__ state, size_t slot_stride) {
  ib::pdl_wait();   // (no early start of the dependents: see causal_conv_rows_kernel)
  const int halo = taps - 1;
  const int b = blockIdx.x;
  if (b >= T) {
    const int hb = b - T, s = hb / halo, j = hb % halo;
    const int a = seg_start[s], n = seg_start[s + 1] - a;
    if (j < n) return;
    const float* src = ext + ((size_t)a + (size_t)s * halo + j) * H;
    float* dst = state + (size_t)seg_slot[s] * slot_stride + (size_t)(j - n) * H;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) st4(dst + i, ld4(src + i));
    return;
  }
  const int t = b, s = seg_of_token[t];
  const int end = seg_start[s + 1];
  const float* cur = ext + ((size_t)t + (size_t)(s + 1) * halo) * H;
  float* keep = end - t <= halo ? state + (size_t)seg_slot[s] * slot_stride + (size_t)(halo - (end - t)) * H : nullptr;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < taps; j++) y = fma4(ld4(w + (size_t)j * H + i), ld4(cur + (ptrdiff_t)(j - halo) * H + i), y);
    const float4 h = ld4(cur + i);
    st4(out + (size_t)t * H + i, add4(h, y));
    if (keep) st4(keep + i, h);
  }
}

template <typename O, bool VEC>
__global__ void __launch_bounds__(kLnThreads) add_layernorm_conv_single_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride,
                                                                               const float* __restrict__ dscale, const float* __restrict__ dbias,
                                                                               const float* __restrict__ w, float eps, float* __restrict__ x_copy,
                                                                               const float* __restrict__ cw, int taps, O* __restrict__ out, int H,
                                                                               const int* __restrict__ seg_slot, float* __restrict__ state, size_t slot_stride) {
  // Row t is segment t (one token each). As in causal_conv_rows_kernel the dependents do not start early. The row's sums are taken in the
  // order of add_layernorm's kernels (the 16-byte form where that one runs, else the scalar form), so a
  // decoded token's normed row has the same bits whichever kernel made it.
  extern __shared__ __align__(16) float row[];
  __shared__ float scratch[32];
  ib::pdl_wait();
  const int t = blockIdx.x, halo = taps - 1;
  float* xr = x + (size_t)t * H;
  auto value = [&](int i) {
    float v = xr[i];
    if (P > 0 || dbias) {
      float d = dbias ? dbias[i] : 0.f;
      if (P > 0) {
        float a = delta[(size_t)t * H + i];
        for (int p = 1; p < P; p++) a += delta[p * delta_stride + (size_t)t * H + i];
        d = dbias ? a + d : a;
      }
      v = dscale ? __fmaf_rn(dscale[i], d, v) : v + d;
      xr[i] = v;
    }
    if (x_copy) x_copy[(size_t)t * H + i] = v;
    row[i] = v;
    return v;
  };
  float* st = state + (size_t)seg_slot[t] * slot_stride;
  if constexpr (VEC) {   // 16-byte accesses; every sum in the order of add_layernorm_vec_kernel and causal_conv_rows_vec_kernel
    float sum = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      float4 v = ld4(xr + i);
      if (P > 0 || dbias) {
        float4 d = dbias ? ld4(dbias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (P > 0) {
          float4 a = ld4(delta + (size_t)t * H + i);
          for (int p = 1; p < P; p++) a = add4(a, ld4(delta + p * delta_stride + (size_t)t * H + i));
          d = dbias ? add4(a, d) : a;
        }
        v = dscale ? fma4(ld4(dscale + i), d, v) : add4(v, d);
        st4(xr + i, v);
      }
      if (x_copy) st4(x_copy + (size_t)t * H + i, v);
      st4(row + i, v);
      sum += (v.x + v.y) + (v.z + v.w);
    }
    const float mean = ib::block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 v = ld4(row + i);
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, e = v.w - mean;
      sq = __fmaf_rn(e, e, __fmaf_rn(c, c, __fmaf_rn(b, b, __fmaf_rn(a, a, sq))));
    }
    const float inv = rsqrtf(ib::block_sum(sq, scratch) / (float)H + eps);
    for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
      const float4 v = ld4(row + i), g = ld4(w + i);
      const float4 h = make_float4((v.x - mean) * inv * g.x, (v.y - mean) * inv * g.y, (v.z - mean) * inv * g.z, (v.w - mean) * inv * g.w);
      float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < halo; j++) {
        const float4 old = ld4(st + (size_t)j * H + i);
        y = fma4(ld4(cw + (size_t)j * H + i), old, y);
        if (j > 0) st4(st + (size_t)(j - 1) * H + i, old);
      }
      y = fma4(ld4(cw + (size_t)halo * H + i), h, y);
      if (halo > 0) st4(st + (size_t)(halo - 1) * H + i, h);
      st4(out + (size_t)t * H + i, add4(h, y));
    }
    return;
  }
  float sum = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) sum += value(i);
  const float mean = ib::block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float c = row[i] - mean;
    sq = __fmaf_rn(c, c, sq);
  }
  const float inv = rsqrtf(ib::block_sum(sq, scratch) / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float h = (row[i] - mean) * inv * w[i];
    float y = 0.f;
    for (int j = 0; j < halo; j++) {
      const float old = st[(size_t)j * H + i];
      y = __fmaf_rn(cw[(size_t)j * H + i], old, y);
      if (j > 0) st[(size_t)(j - 1) * H + i] = old;
    }
    y = __fmaf_rn(cw[(size_t)halo * H + i], h, y);
    if (halo > 0) st[(size_t)(halo - 1) * H + i] = h;
    out[(size_t)t * H + i] = ib::from_f32<O>(h + y);
  }
}


__global__ void depth_average_vec_kernel(float* __restrict__ x, const float* __restrict__ delta, int P, size_t delta_stride, const float* __restrict__ dscale,
                                         const float* __restrict__ dbias, float* __restrict__ stack, size_t layer_stride, int k, const float* __restrict__ mix, int H) {
  ib::pdl_wait();   // (no early start of the dependents: see depth_average_kernel)
  const size_t t = blockIdx.y;
  for (int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4; i < H; i += gridDim.x * blockDim.x * 4) {
    const size_t at = t * H + i;
    float4 v = ld4(x + at);
    if (P > 0) {
      float4 a = ld4(delta + at);
      for (int p = 1; p < P; p++) a = add4(a, ld4(delta + p * delta_stride + at));
      if (dbias) a = add4(a, ld4(dbias + i));
      v = dscale ? fma4(ld4(dscale + i), a, v) : add4(v, a);
    }
    st4(stack + (size_t)k * layer_stride + at, v);
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j < k; j++) {
      const float c = mix[j];
      m = fma4(make_float4(c, c, c, c), ld4(stack + (size_t)j * layer_stride + at), m);
    }
    const float c = mix[k];
    st4(x + at, fma4(make_float4(c, c, c, c), v, m));
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
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = H % 4 == 0 && al(x) && al(delta) && delta_stride % 4 == 0 && al(dscale) && al(dbias) && al(w) && al(out) && al(x_copy) && al(state) && slot_stride % 4 == 0;
  if (out_dtype != IB_F32 && out_dtype != IB_BF16) return ib_set_error("add_layernorm: unknown output dtype %d", out_dtype);
  if (vec && out_dtype == IB_F32) go(add_layernorm_vec_kernel<float>, (float*)out);
  else if (vec) go(add_layernorm_vec_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
  else if (out_dtype == IB_F32) go(add_layernorm_kernel<float>, (float*)out);
  else go(add_layernorm_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
  IB_CHECK_LAUNCH("add_layernorm");
  return 0;
}

extern "C" int ib_add_layernorm_conv_single(float* x, const float* delta, int P, long long delta_stride, const float* dscale, const float* dbias, const float* w,
                                            float eps, float* x_copy, const float* cw, int taps, void* out, int out_dtype, int T, int H, const int* seg_slot, float* state,
                                            long long slot_stride, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && P >= 0 && taps >= 1, "add_layernorm_conv_single: bad sizes T=%d H=%d P=%d taps=%d", T, H, P, taps);
  const size_t smem = (size_t)H * sizeof(float);
  IB_CHECK_ARG(smem <= 200 * 1024, "add_layernorm_conv_single: rows of %d values do not fit in shared memory", H);
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ib::launch(kernel, (unsigned)T, kLnThreads, smem, stream, x, delta, P, (size_t)delta_stride, dscale, dbias, w, eps, x_copy, cw, taps, o, H, seg_slot, state,
               (size_t)slot_stride);
  };
  auto al = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = H % 4 == 0 && al(x) && al(delta) && delta_stride % 4 == 0 && al(dscale) && al(dbias) && al(w) && al(out) && al(x_copy) && al(state) && slot_stride % 4 == 0 &&
                   al(cw);
  if (out_dtype != IB_F32 && out_dtype != IB_BF16) return ib_set_error("add_layernorm_conv_single: unknown output dtype %d", out_dtype);
  if (vec && out_dtype == IB_F32) go(add_layernorm_conv_single_kernel<float, true>, (float*)out);
  else if (vec) go(add_layernorm_conv_single_kernel<__nv_bfloat16, true>, (__nv_bfloat16*)out);
  else if (out_dtype == IB_F32) go(add_layernorm_conv_single_kernel<float, false>, (float*)out);
  else go(add_layernorm_conv_single_kernel<__nv_bfloat16, false>, (__nv_bfloat16*)out);
  IB_CHECK_LAUNCH("add_layernorm_conv_single");
  return 0;
}

extern "C" int ib_causal_conv_rows(const float* ext, const float* w, int taps, void* out, int out_dtype, int T, int H, const int* seg_of_token, const int* seg_start,
                                   const int* seg_slot, int n_segments, float* state, long long slot_stride, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && taps >= 1 && n_segments > 0, "causal_conv_rows: bad sizes T=%d H=%d taps=%d segments=%d", T, H, taps, n_segments);
  const unsigned grid = (unsigned)T + (unsigned)((taps - 1) * n_segments);
  const bool vec = H % 4 == 0 && ((uintptr_t)ext & 15) == 0 && ((uintptr_t)out & 15) == 0 && ((uintptr_t)state & 15) == 0 && slot_stride % 4 == 0 &&
                   ((uintptr_t)w & 15) == 0;
  if (out_dtype != IB_F32 && out_dtype != IB_BF16) return ib_set_error("causal_conv_rows: unknown output dtype %d", out_dtype);
  auto go = [&](auto kernel, auto* o) { ib::launch(kernel, grid, kLnThreads, 0, stream, ext, w, taps, o, T, H, seg_of_token, seg_start, seg_slot, state, (size_t)slot_stride); };
  if (vec && out_dtype == IB_F32) go(causal_conv_rows_vec_kernel<float>, (float*)out);
  else if (vec) go(causal_conv_rows_vec_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
  else if (out_dtype == IB_F32) go(causal_conv_rows_kernel<float>, (float*)out);
  else go(causal_conv_rows_kernel<__nv_bfloat16>, (__nv_bfloat16*)out);
  IB_CHECK_LAUNCH("causal_conv_rows");
  return 0;
}

extern "C" int ib_depth_average(float* x, const float* delta, int P, long long delta_stride, const float* dscale, const float* dbias, float* stack, long long layer_stride, int k,
                                const float* mix, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  IB_CHECK_ARG(T > 0 && H > 0 && k >= 1 && P >= 0, "depth_average: bad sizes T=%d H=%d k=%d P=%d", T, H, k, P);
  IB_CHECK_ARG(T <= 65535, "depth_average: T=%d rows exceed the grid limit 65535", T);
  const bool vec = H % 4 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)delta & 15) == 0 && delta_stride % 4 == 0 && ((uintptr_t)dscale & 15) == 0 &&
                   ((uintptr_t)dbias & 15) == 0 && ((uintptr_t)stack & 15) == 0 && layer_stride % 4 == 0;
  if (vec)
    ib::launch(depth_average_vec_kernel, dim3(min((H / 4 + 255) / 256, 32), T), 256, 0, stream, x, delta, P, (size_t)delta_stride, dscale, dbias, stack, (size_t)layer_stride, k,
               mix, H);
  else
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
