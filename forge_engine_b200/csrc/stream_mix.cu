// Residual streams, their norms, and small token-wise kernels of layers built on them.
//
// stream_mix_norm: the residual stream exists in S copies x_1..x_S per token (S = 1: the
// usual single stream).  One launch does, per token and all in 32-bit,
//   x'_t = sum_s mix[s, t] x_s + c * out[t] * y          (y: the last sublayer's output)
//   u    = sum_t in[t] x'_t
//   z    = norm(u) * w                                   (RMS or layer norm, or none)
// with every piece optional: no y (nothing to add), no mix (identity), no out / in (ones).
// It is the fused "add the update, then normalise for the next sublayer" of a pre-norm
// block, generalised to several streams and to a layer norm.
//
// act_mul: act(gate) * up for a row [gate | up]; gated_rmsnorm: rms(x) * w * sigmoid(g).
#include "common.cuh"

#define FE_MAX_STREAMS 16
#define FE_VEC_STREAMS 8      // the 16-byte form keeps four elements of every stream in registers
#define FE_NORM_NONE 0
#define FE_NORM_RMS 1
#define FE_NORM_LAYER 2

template <typename TU, typename TO>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(float* __restrict__ streams, int S, const TU* __restrict__ update, float update_scale,
                       const float* __restrict__ mix, const float* __restrict__ out_coef,
                       const float* __restrict__ in_coef, int norm_kind, const float* __restrict__ weight,
                       float eps, TO* __restrict__ out, const int* __restrict__ row_map, int W,
                       int write_streams) {
  extern __shared__ float u_row[];          // [W]
  __shared__ float scratch[33];
  __shared__ float c_mix[FE_MAX_STREAMS * FE_MAX_STREAMS], c_out[FE_MAX_STREAMS], c_in[FE_MAX_STREAMS];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_map ? row_map[r] : r;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) c_mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = (out_coef ? out_coef[threadIdx.x] : 1.f) * update_scale;
    c_in[threadIdx.x] = in_coef ? in_coef[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* base = streams + (size_t)src * S * W;
  const TU* upd = update ? update + (size_t)src * W : nullptr;
  float total = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float x[FE_MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < FE_MAX_STREAMS; ++s) x[s] = s < S ? base[(size_t)s * W + i] : 0.f;
    float u = 0.f;
    if (upd) {
      const float y = to_float(upd[i]);
#pragma unroll
      for (int t = 0; t < FE_MAX_STREAMS; ++t) {
        if (t < S) {
          float v = 0.f;
#pragma unroll
          for (int s = 0; s < FE_MAX_STREAMS; ++s)
            if (s < S) v = fmaf(c_mix[s * S + t], x[s], v);
          v = fmaf(c_out[t], y, v);
          if (write_streams) base[(size_t)t * W + i] = v;
          u = fmaf(c_in[t], v, u);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < FE_MAX_STREAMS; ++t)
        if (t < S) u = fmaf(c_in[t], x[t], u);
    }
    u_row[i] = u;
    total += norm_kind == FE_NORM_RMS ? u * u : u;
  }
  if (out == nullptr || norm_kind == FE_NORM_NONE) {
    if (out != nullptr)
      for (int i = threadIdx.x; i < W; i += blockDim.x) out[(size_t)r * W + i] = from_float<TO>(u_row[i]);
    return;
  }
  total = block_sum(total, scratch);
  float mean = 0.f, inv;
  if (norm_kind == FE_NORM_RMS) {
    inv = 1.f / sqrtf(total / (float)W + eps);
  } else {
    mean = total / (float)W;
    float dev = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float d = u_row[i] - mean;
      dev = fmaf(d, d, dev);
    }
    dev = block_sum(dev, scratch);
    inv = 1.f / sqrtf(dev / (float)W + eps);
  }
  TO* dst = out + (size_t)r * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = from_float<TO>((u_row[i] - mean) * inv * weight[i]);
}

// The same for widths that are multiples of 4 (and 16-byte aligned rows): a thread handles four
// neighbouring elements of every stream with 16-byte loads and stores; same arithmetic, same
// order of sums.
template <typename TU, typename TO>
__global__ void __launch_bounds__(256)
stream_mix_norm_vec_kernel(float* __restrict__ streams, int S, const TU* __restrict__ update, float update_scale,
                           const float* __restrict__ mix, const float* __restrict__ out_coef,
                           const float* __restrict__ in_coef, int norm_kind, const float* __restrict__ weight,
                           float eps, TO* __restrict__ out, const int* __restrict__ row_map, int W,
                           int write_streams) {
  extern __shared__ float u_row[];          // [W]
  __shared__ float scratch[33];
  __shared__ float c_mix[FE_VEC_STREAMS * FE_VEC_STREAMS], c_out[FE_VEC_STREAMS], c_in[FE_VEC_STREAMS];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_map ? row_map[r] : r;
  for (int i = threadIdx.x; i < S * S; i += blockDim.x) c_mix[i] = mix ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
  if (threadIdx.x < S) {
    c_out[threadIdx.x] = (out_coef ? out_coef[threadIdx.x] : 1.f) * update_scale;
    c_in[threadIdx.x] = in_coef ? in_coef[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* base = streams + (size_t)src * S * W;
  const TU* upd = update ? update + (size_t)src * W : nullptr;
  float total = 0.f;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    float x[FE_VEC_STREAMS][4];
#pragma unroll
    for (int s = 0; s < FE_VEC_STREAMS; ++s)
      if (s < S) load4(base + (size_t)s * W + i, x[s]);
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    if (upd) {
      float y[4];
      load4(upd + i, y);
#pragma unroll
      for (int t = 0; t < FE_VEC_STREAMS; ++t) {
        if (t < S) {
          float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int s = 0; s < FE_VEC_STREAMS; ++s)
            if (s < S) {
#pragma unroll
              for (int e = 0; e < 4; ++e) v[e] = fmaf(c_mix[s * S + t], x[s][e], v[e]);
            }
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[e] = fmaf(c_out[t], y[e], v[e]);
            u[e] = fmaf(c_in[t], v[e], u[e]);
          }
          if (write_streams) store4(base + (size_t)t * W + i, v);
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < FE_VEC_STREAMS; ++t)
        if (t < S) {
#pragma unroll
          for (int e = 0; e < 4; ++e) u[e] = fmaf(c_in[t], x[t][e], u[e]);
        }
    }
    store4(u_row + i, u);
#pragma unroll
    for (int e = 0; e < 4; ++e) total += norm_kind == FE_NORM_RMS ? u[e] * u[e] : u[e];
  }
  if (out == nullptr) return;
  float mean = 0.f, inv = 1.f;
  if (norm_kind != FE_NORM_NONE) {
    total = block_sum(total, scratch);
    if (norm_kind == FE_NORM_RMS) {
      inv = 1.f / sqrtf(total / (float)W + eps);
    } else {
      mean = total / (float)W;
      float dev = 0.f;
      for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float d = u_row[i + e] - mean;
          dev = fmaf(d, d, dev);
        }
      }
      dev = block_sum(dev, scratch);
      inv = 1.f / sqrtf(dev / (float)W + eps);
    }
  }
  TO* dst = out + (size_t)r * W;
  for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
    float y[4], w[4] = {1.f, 1.f, 1.f, 1.f};
    if (norm_kind != FE_NORM_NONE) load4(weight + i, w);
#pragma unroll
    for (int e = 0; e < 4; ++e) y[e] = norm_kind == FE_NORM_NONE ? u_row[i + e] : (u_row[i + e] - mean) * inv * w[e];
    store4(dst + i, y);
  }
}

FE_EXPORT int fe_stream_mix_norm(float* streams, int n_streams, const void* update, int update_dtype,
                                 float update_scale, const float* mix, const float* out_coef, const float* in_coef,
                                 int norm_kind, const float* weight, float eps, void* out, int out_dtype,
                                 const int* row_map, int rows, int width, int write_streams, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (n_streams < 1 || n_streams > FE_MAX_STREAMS || width < 1) return FE_ERR_BAD_SHAPE;
  if (norm_kind != FE_NORM_NONE && out != nullptr && weight == nullptr) return FE_ERR_BAD_SHAPE;
  const size_t smem = sizeof(float) * (size_t)width;
  if (smem > 200 * 1024) return FE_ERR_TOO_LARGE;
  int threads = width >= 2048 ? 256 : 128;
  int rc = 0;
  const int update_bytes = update_dtype == FE_DTYPE_F32 ? 16 : 8, out_bytes = out_dtype == FE_DTYPE_F32 ? 16 : 8;
  const bool vec = n_streams <= FE_VEC_STREAMS && (width % 4) == 0 && ((uintptr_t)streams % 16) == 0 && ((uintptr_t)weight % 16) == 0 &&
                   ((uintptr_t)update % update_bytes) == 0 && ((uintptr_t)out % out_bytes) == 0;
  if (vec) threads = width >= 1024 ? 256 : width >= 512 ? 128 : 64;
#define LAUNCH(TU, TO)                                                                                          \
  do {                                                                                                          \
    auto kernel = vec ? stream_mix_norm_vec_kernel<TU, TO> : stream_mix_norm_kernel<TU, TO>;                    \
    if (smem > 48 * 1024)                                                                                       \
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                     \
    rc = fe_launch_dependent(kernel, dim3(rows), dim3(threads), smem, stream, streams,                          \
                             n_streams, (const TU*)update, update_scale, mix, out_coef, in_coef, norm_kind,     \
                             weight, eps, (TO*)out, row_map, width, write_streams);                             \
  } while (0)
  const int ud = update ? update_dtype : FE_DTYPE_F32;
  if (ud == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32) LAUNCH(float, float);
  else if (ud == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16) LAUNCH(bf16, bf16);
  else if (ud == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16) LAUNCH(float, bf16);
  else if (ud == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_F32) LAUNCH(bf16, float);
  else return FE_ERR_BAD_DTYPE;
#undef LAUNCH
  return rc ? rc : fe_last_error();
}

// ---------------------------------------------------------------------------
// out[n, i] = act(gate_up[n, i]) * gate_up[n, inter + i];  act 0: SiLU, 1: the tanh form of GELU,
// 2: the clamped unit g' sigmoid(slope g') (u' + 1) with g' = min(g, limit), u' = clamp(u, +-limit)
// ---------------------------------------------------------------------------
struct ActParams { int act; float limit, slope; };

__device__ __forceinline__ float act_apply(float z, float u, const ActParams& a) {
  if (a.act == 0) return z / (1.f + expf(-z)) * u;
  if (a.act == 2) {
    const float g = fminf(z, a.limit);
    const float v = fminf(fmaxf(u, -a.limit), a.limit);
    return g / (1.f + expf(-a.slope * g)) * (v + 1.f);
  }
  const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.f + tanhf(inner)) * u;
}

// block == 0: a row is [all gate | all up]; block == B > 0: it alternates B gate features, B up
// features (the layout the fused projection kernels want).
__device__ __forceinline__ void gate_up_at(int i, int inter, int block, int* gate_at, int* up_at) {
  if (block == 0) { *gate_at = i; *up_at = inter + i; }
  else { const int b = i / block; *gate_at = 2 * b * block + (i - b * block); *up_at = *gate_at + block; }
}

template <typename TI, typename TO>
__global__ void act_mul_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inter, ActParams act, int block) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const TI* g = gate_up + (size_t)row * 2 * inter;
  TO* o = out + (size_t)row * inter;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < inter; i += gridDim.y * blockDim.x) {
    int ga, ua;
    gate_up_at(i, inter, block, &ga, &ua);
    o[i] = from_float<TO>(act_apply(to_float(g[ga]), to_float(g[ua]), act));
  }
}

template <typename TI, typename TO>
__global__ void act_mul_vec_kernel(const TI* __restrict__ gate_up, TO* __restrict__ out, int inter, ActParams act, int block) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const TI* g = gate_up + (size_t)row * 2 * inter;
  TO* o = out + (size_t)row * inter;
  for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < inter; i += gridDim.y * blockDim.x * 4) {
    float a[4], b[4];
    int ga, ua;
    gate_up_at(i, inter, block, &ga, &ua);      // block is a multiple of 4: four features stay together
    load4(g + ga, a);
    load4(g + ua, b);
#pragma unroll
    for (int e = 0; e < 4; ++e) a[e] = act_apply(a[e], b[e], act);
    store4(o + i, a);
  }
}

FE_EXPORT int fe_act_mul(const void* gate_up, int in_dtype, void* out, int out_dtype, int rows, int inter, int act_kind,
                         int block, float limit, float slope, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (act_kind < 0 || act_kind > 2) return FE_ERR_BAD_SHAPE;
  const ActParams act{act_kind, limit, slope};
  if (block < 0 || (block > 0 && (inter % block) != 0)) return FE_ERR_BAD_SHAPE;
  const int threads = 256;
  if ((inter % 4) == 0 && (block % 4) == 0 && ((uintptr_t)gate_up % 16) == 0 && ((uintptr_t)out % 16) == 0) {
    int pieces = (inter / 4 + threads - 1) / threads;
    if (pieces > 64) pieces = 64;
    dim3 vgrid(rows, pieces);
    if (in_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32)
      return fe_launch_dependent(act_mul_vec_kernel<float, float>, vgrid, dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, act, block);
    if (in_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16)
      return fe_launch_dependent(act_mul_vec_kernel<bf16, bf16>, vgrid, dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, act, block);
    if (in_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16)
      return fe_launch_dependent(act_mul_vec_kernel<float, bf16>, vgrid, dim3(threads), 0, stream, (const float*)gate_up, (bf16*)out, inter, act, block);
    return FE_ERR_BAD_DTYPE;
  }
  int chunks = (inter + threads - 1) / threads;
  if (chunks > 64) chunks = 64;
  dim3 grid(rows, chunks);
  if (in_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32)
    return fe_launch_dependent(act_mul_kernel<float, float>, grid, dim3(threads), 0, stream, (const float*)gate_up, (float*)out, inter, act, block);
  if (in_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(act_mul_kernel<bf16, bf16>, grid, dim3(threads), 0, stream, (const bf16*)gate_up, (bf16*)out, inter, act, block);
  if (in_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(act_mul_kernel<float, bf16>, grid, dim3(threads), 0, stream, (const float*)gate_up, (bf16*)out, inter, act, block);
  return FE_ERR_BAD_DTYPE;
}

// ---------------------------------------------------------------------------
// out[n, :] = x[n, :] / sqrt(mean(x[n, :]^2) + eps) * weight * sigmoid(gate[n, :])
// x is 32-bit [rows, size]; gate row n starts at gate + n * gate_stride.
// ---------------------------------------------------------------------------
template <typename TG, typename TO>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ x, const TG* __restrict__ gate, int gate_stride,
                                     const float* __restrict__ weight, TO* __restrict__ out, int size, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const float* xr = x + (size_t)r * size;
  const TG* gr = gate + (size_t)r * gate_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
  const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)size + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float g = to_float(gr[i]);
    out[(size_t)r * size + i] = from_float<TO>(xr[i] * inv * weight[i] * (1.f / (1.f + expf(-g))));
  }
}

FE_EXPORT int fe_gated_rmsnorm(const float* x, const void* gate, int gate_dtype, int gate_stride, const float* weight,
                               void* out, int out_dtype, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = size >= 1024 ? 256 : 128;
  if (gate_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_F32)
    return fe_launch_dependent(gated_rmsnorm_kernel<float, float>, dim3(rows), dim3(threads), 0, stream, x, (const float*)gate, gate_stride, weight, (float*)out, size, eps);
  if (gate_dtype == FE_DTYPE_BF16 && out_dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(gated_rmsnorm_kernel<bf16, bf16>, dim3(rows), dim3(threads), 0, stream, x, (const bf16*)gate, gate_stride, weight, (bf16*)out, size, eps);
  if (gate_dtype == FE_DTYPE_F32 && out_dtype == FE_DTYPE_BF16)
    return fe_launch_dependent(gated_rmsnorm_kernel<float, bf16>, dim3(rows), dim3(threads), 0, stream, x, (const float*)gate, gate_stride, weight, (bf16*)out, size, eps);
  return FE_ERR_BAD_DTYPE;
}
