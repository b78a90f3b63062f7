// Row-wise kernels for designs whose residual stream travels in several copies ("streams") and whose
// embedding adds a row of a second table chosen by the token and the token before it.
//
//   srb_embedding_pairs   x[r] = table[id_r] * scale + pairs[f(id_(r-1), id_r)], written `copies` times
//   srb_remember_tokens   last[slot of request q] = the last token id that q brought in this step
//   srb_stream_step       the update of the copies by a sublayer's result, the read of the next sublayer's
//                         input from the copies and its RMS norm, in one pass over the row
//   srb_softcap           v <- cap * tanh(v / cap)
//   srb_activate          out = act(x) for a feed-forward without a gate
//
// All arithmetic is 32-bit; T is the storage type of tables and activations.
#include "common.cuh"
#include "activations.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

// The row of the pair table: (previous * mul_prev + current * mul_cur) mod buckets, or row `buckets` for a
// sequence's first token.  The previous token of a request's first row of this step is what the request's state
// slot remembers; inside the step it is the row before.
template <typename T>
__global__ void embedding_pairs_kernel(const int* __restrict__ ids, const int* __restrict__ positions,
                                       const int* __restrict__ row_request, const int* __restrict__ cu_rows,
                                       const int* __restrict__ state_slots, const int* __restrict__ last_token,
                                       const T* __restrict__ table, const T* __restrict__ pairs,
                                       float* __restrict__ out, int width, int vocab, int copies, long long buckets,
                                       long long mul_prev, long long mul_cur, float scale, int* error_word) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const int id = ids[row];
  const bool bad = id < 0 || id >= vocab;
  if (bad && threadIdx.x == 0) atomicOr(error_word, SRB_FLAG_BAD_TOKEN);
  long long pair_row = buckets;
  if (pairs && positions[row] > 0) {
    const int request = row_request[row];
    int previous = row > cu_rows[request] ? ids[row - 1] : last_token[state_slots[request]];
    if (previous < 0 || previous >= vocab) {
      if (threadIdx.x == 0) atomicOr(error_word, SRB_FLAG_BAD_TOKEN);
      previous = 0;
    }
    pair_row = ((long long)previous * mul_prev + (long long)(bad ? 0 : id) * mul_cur) % buckets;
    if (pair_row < 0) pair_row += buckets;
  }
  const T* src = table + (size_t)(bad ? 0 : id) * width;
  const T* add = pairs ? pairs + (size_t)pair_row * width : nullptr;
  float* dst = out + (size_t)row * copies * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float v = bad ? 0.f : srb_to_float(src[i]) * scale;
    if (add) v += srb_to_float(add[i]);
    for (int c = 0; c < copies; ++c) dst[(size_t)c * width + i] = v;
  }
}

extern "C" int srb_embedding_pairs(const int* ids, const int* positions, const int* row_request, const int* cu_rows,
                                   const int* state_slots, const int* last_token, const void* table, const void* pairs,
                                   float* out, int rows, int width, int vocab, int copies, long long buckets,
                                   long long mul_prev, long long mul_cur, float scale, int* error_word, int dtype,
                                   void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0 || vocab <= 0 || copies <= 0) SRB_FAIL("embedding_pairs: width, vocabulary and copies must be positive");
  if (pairs && (buckets <= 0 || !positions || !row_request || !cu_rows || !state_slots || !last_token))
    SRB_FAIL("embedding_pairs: a pair table needs its bucket count, the step's index arrays and the remembered tokens");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(embedding_pairs_kernel<float>, dim3(rows), dim3(256), 0, s, ids, positions, row_request,
                             cu_rows, state_slots, last_token, (const float*)table, (const float*)pairs, out, width, vocab,
                             copies, buckets, mul_prev, mul_cur, scale, error_word));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(embedding_pairs_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, ids, positions,
                             row_request, cu_rows, state_slots, last_token, (const __nv_bfloat16*)table,
                             (const __nv_bfloat16*)pairs, out, width, vocab, copies, buckets, mul_prev, mul_cur, scale,
                             error_word));
  else
    SRB_FAIL("embedding_pairs: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("embedding_pairs");
  return SRB_OK;
}

// A kernel of its own, after the embedding: the first row of a request reads the slot that its last row writes.
__global__ void remember_tokens_kernel(const int* __restrict__ ids, const int* __restrict__ cu_rows,
                                       const int* __restrict__ state_slots, int* __restrict__ last_token, int requests) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int request = blockIdx.x * blockDim.x + threadIdx.x;
  if (request >= requests) return;
  const int end = cu_rows[request + 1];
  if (end > cu_rows[request]) last_token[state_slots[request]] = ids[end - 1];
}

extern "C" int srb_remember_tokens(const int* ids, const int* cu_rows, const int* state_slots, int* last_token,
                                   int requests, void* stream) {
  if (requests <= 0) return SRB_OK;
  SRB_CUDA_CALL(srb_launch(remember_tokens_kernel, dim3((requests + 127) / 128), dim3(128), 0, (cudaStream_t)stream, ids,
                           cu_rows, state_slots, last_token, requests));
  SRB_LAUNCH_CHECK("remember_tokens");
  return SRB_OK;
}

// ---- copies of the residual stream -----------------------------------------------------------------------
// x: float [rows, S, width].  With a pending result y of the sublayer before (T [rows, width], or `parts` float
// partial sums `part_stride` elements apart, added in order), every copy is replaced, all at once from the old ones:
//     x_t <- sum_s mix[s, t] x_s + spread[t] * y          (mix is [from, to])
// Then, if an output is wanted: u = sum_t gather[t] x_t, out = u / sqrt(mean(u^2) + eps) * weight.  `row_index`
// picks rows (the copies are then left as they are in memory: the update is applied on the fly).
#define STREAMS_MAX 8

struct StreamStepArgs {
  float* x;
  const void* y;             // T, or null
  const float* y_parts;      // float partial sums, or null
  int parts;
  long long part_stride;
  const float* mix;          // [S, S] or null (no pending update)
  const float* spread;       // [S]
  const float* gather;       // [S] or null (no output)
  const float* weight;       // [width] or null: no scaling
  float eps;
  void* out;                 // T [rows_out, out_pitch]
  long long out_pitch;
  const int* row_index;
  int streams, width, write_back, norm;
};

// four (VEC) or one consecutive columns of the result of the sublayer before, as floats
template <typename T, int VEC>
__device__ __forceinline__ void stream_load_result(const StreamStepArgs& a, const T* y, size_t row_offset, int i, float (&r)[VEC]) {
#pragma unroll
  for (int v = 0; v < VEC; ++v) r[v] = 0.f;
  if (y) {
    if (VEC == 4 && sizeof(T) == 2) {
      const uint2 raw = *reinterpret_cast<const uint2*>(y + i);
      const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
      const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
      r[0] = lo.x; r[1] = lo.y; r[VEC - 2] = hi.x; r[VEC - 1] = hi.y;
    } else if (VEC == 4) {
      const float4 raw = *reinterpret_cast<const float4*>(y + i);
      r[0] = raw.x; r[1] = raw.y; r[VEC - 2] = raw.z; r[VEC - 1] = raw.w;
    } else {
      r[0] = srb_to_float(y[i]);
    }
  }
  for (int part = 0; part < a.parts; ++part) {
    const float* p = a.y_parts + part * a.part_stride + row_offset + i;
    if (VEC == 4) {
      const float4 raw = *reinterpret_cast<const float4*>(p);
      r[0] += raw.x; r[1] += raw.y; r[VEC - 2] += raw.z; r[VEC - 1] += raw.w;
    } else {
      r[0] += *p;
    }
  }
}

// VEC 4: the row's width is a multiple of four and every pointer is 16-byte aligned; a thread moves four columns at a time.
template <typename T, int VEC>
__global__ void stream_step_kernel(StreamStepArgs a) {
  extern __shared__ __align__(16) float staged[];      // [width]: u of this row
  __shared__ float reduce[33];
  __shared__ float coef[STREAMS_MAX * STREAMS_MAX + 2 * STREAMS_MAX];
  srb_launch_dependents();
  const int S = a.streams;
  float* mix = coef;
  float* spread = coef + STREAMS_MAX * STREAMS_MAX;
  float* gather = spread + STREAMS_MAX;
  if (threadIdx.x < S * S) mix[threadIdx.x] = a.mix ? a.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    spread[threadIdx.x] = a.mix ? a.spread[threadIdx.x] : 0.f;
    gather[threadIdx.x] = a.gather ? a.gather[threadIdx.x] : 0.f;
  }
  srb_grid_dependency_wait();
  __syncthreads();
  const int src = a.row_index ? a.row_index[blockIdx.x] : blockIdx.x;
  float* x = a.x + (size_t)src * S * a.width;
  const size_t row_offset = (size_t)src * a.width;
  const T* y = a.y ? reinterpret_cast<const T*>(a.y) + row_offset : nullptr;
  float squares = 0.f;
  for (int i = threadIdx.x * VEC; i < a.width; i += blockDim.x * VEC) {
    float old[STREAMS_MAX][VEC], u[VEC];
#pragma unroll
    for (int s = 0; s < STREAMS_MAX; ++s) {
      if (s < S) {
        if (VEC == 4) {
          const float4 raw = *reinterpret_cast<const float4*>(x + (size_t)s * a.width + i);
          old[s][0] = raw.x; old[s][1] = raw.y; old[s][VEC - 2] = raw.z; old[s][VEC - 1] = raw.w;
        } else {
          old[s][0] = x[(size_t)s * a.width + i];
        }
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) u[v] = 0.f;
    if (a.mix) {
      float result[VEC];
      stream_load_result<T, VEC>(a, y, row_offset, i, result);
#pragma unroll
      for (int t = 0; t < STREAMS_MAX; ++t) {
        if (t < S) {
          float fresh[VEC];
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            float sum = 0.f;
#pragma unroll
            for (int s = 0; s < STREAMS_MAX; ++s)
              if (s < S) sum = fmaf(mix[s * S + t], old[s][v], sum);
            fresh[v] = fmaf(spread[t], result[v], sum);
            u[v] = fmaf(gather[t], fresh[v], u[v]);
          }
          if (a.write_back) {
            if (VEC == 4)
              *reinterpret_cast<float4*>(x + (size_t)t * a.width + i) = make_float4(fresh[0], fresh[1], fresh[VEC - 2], fresh[VEC - 1]);
            else
              x[(size_t)t * a.width + i] = fresh[0];
          }
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < STREAMS_MAX; ++t)
        if (t < S) {
#pragma unroll
          for (int v = 0; v < VEC; ++v) u[v] = fmaf(gather[t], old[t][v], u[v]);
        }
    }
    if (a.gather) {
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        staged[i + v] = u[v];
        squares = fmaf(u[v], u[v], squares);
      }
    }
  }
  if (!a.gather) return;
  float inv = 1.f;
  if (a.norm) {
    const float total = srb_block_sum(squares, reduce);
    inv = rsqrtf(total / (float)a.width + a.eps);
  } else {
    __syncthreads();
  }
  T* out = reinterpret_cast<T*>(a.out) + (size_t)blockIdx.x * a.out_pitch;
  for (int i = threadIdx.x * VEC; i < a.width; i += blockDim.x * VEC) {
    float v[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) v[k] = staged[i + k] * inv * (a.weight ? a.weight[i + k] : 1.f);
    if (VEC == 4 && sizeof(T) == 2) {
      uint2 raw;
      *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v[0], v[1]);
      *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v[VEC - 2], v[VEC - 1]);
      *reinterpret_cast<uint2*>(out + i) = raw;
    } else {
#pragma unroll
      for (int k = 0; k < VEC; ++k) out[i + k] = srb_from_float<T>(v[k]);
    }
  }
}

extern "C" int srb_stream_step(float* x, const void* y, const float* y_parts, int parts, long long part_stride,
                               const float* mix, const float* spread, const float* gather, const float* weight, float eps,
                               int norm, void* out, long long out_pitch, const int* row_index, int rows, int streams,
                               int width, int write_back, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (streams <= 0 || streams > STREAMS_MAX) SRB_FAIL("stream_step: %d copies of the stream; 1 to %d are taken", streams, STREAMS_MAX);
  if (width <= 0) SRB_FAIL("stream_step: width %d must be positive", width);
  if (mix && !spread) SRB_FAIL("stream_step: an update needs the weights of the result");
  if (mix && !y && parts <= 0) SRB_FAIL("stream_step: an update needs a result");
  if (gather && !out) SRB_FAIL("stream_step: a read needs an output");
  StreamStepArgs a;
  a.x = x; a.y = y; a.y_parts = y_parts; a.parts = y_parts ? parts : 0; a.part_stride = part_stride; a.mix = mix;
  a.spread = spread; a.gather = gather; a.weight = weight; a.eps = eps; a.out = out; a.out_pitch = out_pitch;
  a.row_index = row_index; a.streams = streams; a.width = width; a.write_back = write_back && !row_index; a.norm = norm;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) SRB_FAIL("stream_step: width %d exceeds what a block can stage", width);
  const bool vec = width % 4 == 0 && part_stride % 4 == 0 && out_pitch % 4 == 0 &&
                   (((uintptr_t)x | (uintptr_t)y | (uintptr_t)y_parts | (uintptr_t)out) & 15) == 0;
  const int threads = vec ? (width >= 4096 ? 512 : 256) : (width >= 2048 ? 512 : 256);
  cudaStream_t s = (cudaStream_t)stream;
#define STREAM_STEP_LAUNCH(T, VEC)                                                                                          \
  do {                                                                                                                      \
    if (smem > 48 * 1024)                                                                                                   \
      SRB_CUDA_CALL(cudaFuncSetAttribute(stream_step_kernel<T, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    SRB_CUDA_CALL(srb_launch(stream_step_kernel<T, VEC>, dim3(rows), dim3(threads), smem, s, a));                           \
  } while (0)
  if (dtype == SRB_DTYPE_F32) {
    if (vec) STREAM_STEP_LAUNCH(float, 4); else STREAM_STEP_LAUNCH(float, 1);
  } else if (dtype == SRB_DTYPE_BF16) {
    if (vec) STREAM_STEP_LAUNCH(__nv_bfloat16, 4); else STREAM_STEP_LAUNCH(__nv_bfloat16, 1);
  } else {
    SRB_FAIL("stream_step: unknown dtype %d", dtype);
  }
#undef STREAM_STEP_LAUNCH
  SRB_LAUNCH_CHECK("stream_step");
  return SRB_OK;
}

// ---- element-wise ------------------------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ values, size_t total, float cap) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const float inv = 1.0f / cap;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    values[i] = cap * tanhf(values[i] * inv);
}

extern "C" int srb_softcap(float* values, long long total, float cap, void* stream) {
  if (total <= 0) return SRB_OK;
  if (!(cap > 0.f)) SRB_FAIL("softcap: the cap must be positive");
  size_t blocks = ((size_t)total + 255) / 256;
  const size_t most = (size_t)srb_sm_count() * 16;
  SRB_CUDA_CALL(srb_launch(softcap_kernel, dim3((unsigned)(blocks > most ? most : blocks)), dim3(256), 0,
                           (cudaStream_t)stream, values, (size_t)total, cap));
  SRB_LAUNCH_CHECK("softcap");
  return SRB_OK;
}

template <typename T>
__global__ void activate_kernel(const T* __restrict__ x, T* __restrict__ out, size_t total, int activation) {
  srb_launch_dependents();
  srb_grid_dependency_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
    out[i] = srb_from_float<T>(srb_gated<true>(activation, srb_to_float(x[i]), 1.0f));
}

extern "C" int srb_activate(const void* x, void* out, long long total, int activation, int dtype, void* stream) {
  if (total <= 0) return SRB_OK;
  if (activation < 0 || activation >= SRB_ACT_COUNT) SRB_FAIL("activate: unknown activation %d", activation);
  size_t blocks = ((size_t)total + 255) / 256;
  const size_t most = (size_t)srb_sm_count() * 16;
  const dim3 grid((unsigned)(blocks > most ? most : blocks));
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(activate_kernel<float>, grid, dim3(256), 0, s, (const float*)x, (float*)out, (size_t)total, activation));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(activate_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, (const __nv_bfloat16*)x,
                             (__nv_bfloat16*)out, (size_t)total, activation));
  else
    SRB_FAIL("activate: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("activate");
  return SRB_OK;
}
