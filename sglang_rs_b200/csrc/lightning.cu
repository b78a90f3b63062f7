// Linear attention with one fixed decay per head ("lightning attention") over a state of fixed size per request.
//
// Per head, with q_t, k_t (dim entries) and v_t (vdim entries) the SiLU of the row's projections:
//     S_t = decay * S_(t-1) + k_t v_t^T          S: [dim, vdim] 32-bit floats, zero before a sequence's first token
//     o_t = S_t^T q_t
// The rows of a request in one step (a prompt portion, or one decoded token) are walked in chunks of LA_CHUNK
// tokens.  Inside a chunk that starts from state S and holds tokens 0 .. n-1:
//     A[t, j] = (q_t . k_j) decay^(t - j)                              for j <= t
//     o_t     = sum_(j <= t) A[t, j] v_j + decay^(t+1) S^T q_t
//     S      <- decay^n S + sum_j decay^(n-1-j) k_j v_j^T
// Powers of the decay are products of 32-bit floats, never quotients, so nothing overflows however small the
// decay is.  Scores, weights, sums and the state are 32-bit in both dtypes; T is the type of the projections.
//
//   srb_lightning_scan       the recurrence: reads q, k, v from the rows of the stacked projection, updates the
//                            requests' states in place, writes o as float [rows, heads * vdim]
//   srb_lightning_gate_norm  out = o / sqrt(mean(o^2) + eps) * weight * sigmoid(g), over all heads of a row together
#include "common.cuh"
#include <math.h>

SRB_DEFINE_LAST_ERROR()
SRB_DEFINE_PDL_SWITCH()

#define LA_CHUNK 32
#define LA_THREADS 256
#define LA_SLICE 64          // value columns that one block owns at most

struct LightningArgs {
  const void* proj;          // T [rows, pitch]
  long long pitch;
  int q_offset, k_offset, v_offset;
  const int* cu_rows;        // [requests + 1]
  const int* positions;      // [rows]
  const int* state_slots;    // [requests]
  float* state;              // [slots, heads, dim, vdim]
  const float* decay;        // [heads]
  float* out;                // [rows, heads * vdim]
  int heads, dim, vdim, slices, slice_width, read_only;
};

__device__ __forceinline__ float la_silu(float x) { return x / (1.0f + expf(-x)); }

template <typename T>
__global__ void __launch_bounds__(LA_THREADS) lightning_scan_kernel(LightningArgs a) {
  extern __shared__ float smem[];
  srb_launch_dependents();
  const int head = blockIdx.x / a.slices, slice = blockIdx.x % a.slices;
  const int request = blockIdx.y;
  const int dim = a.dim, c0 = slice * a.slice_width;
  const int vs = min(a.slice_width, a.vdim - c0);
  const int qk_pitch = dim + 1;
  float* S = smem;                                  // [dim][slice_width]
  float* Q = S + dim * a.slice_width;               // [LA_CHUNK][dim + 1]
  float* K = Q + LA_CHUNK * qk_pitch;               // [LA_CHUNK][dim + 1]
  float* V = K + LA_CHUNK * qk_pitch;               // [LA_CHUNK][slice_width]
  float* A = V + LA_CHUNK * a.slice_width;          // [LA_CHUNK][LA_CHUNK + 1]
  float* power = A + LA_CHUNK * (LA_CHUNK + 1);     // [LA_CHUNK + 1]: decay^n
  if (vs <= 0) return;
  if (threadIdx.x == 0) {
    const float decay = a.decay[head];
    float p = 1.f;
    for (int n = 0; n <= LA_CHUNK; ++n) {
      power[n] = p;
      p *= decay;
    }
  }
  srb_grid_dependency_wait();
  const int row_begin = a.cu_rows[request], row_end = a.cu_rows[request + 1];
  if (row_end <= row_begin) return;
  float* state = a.state + (((size_t)a.state_slots[request] * a.heads + head) * dim) * a.vdim + c0;
  const bool fresh = a.positions[row_begin] == 0;    // a sequence's first token starts from the zero state
  for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
    const int d = e / vs, c = e - d * vs;
    S[d * a.slice_width + c] = fresh ? 0.f : state[(size_t)d * a.vdim + c];
  }
  const T* proj = reinterpret_cast<const T*>(a.proj);
  const int out_pitch = a.heads * a.vdim;
  for (int row0 = row_begin; row0 < row_end; row0 += LA_CHUNK) {
    const int n = min(LA_CHUNK, row_end - row0);
    __syncthreads();                                 // the chunk before is done with Q, K, V, A; S is updated
    for (int e = threadIdx.x; e < n * dim; e += LA_THREADS) {
      const int t = e / dim, d = e - t * dim;
      const T* row = proj + (size_t)(row0 + t) * a.pitch + (size_t)head * dim + d;
      Q[t * qk_pitch + d] = la_silu(srb_to_float(row[a.q_offset]));
      K[t * qk_pitch + d] = la_silu(srb_to_float(row[a.k_offset]));
    }
    for (int e = threadIdx.x; e < n * vs; e += LA_THREADS) {
      const int t = e / vs, c = e - t * vs;
      V[t * a.slice_width + c] =
          la_silu(srb_to_float(proj[(size_t)(row0 + t) * a.pitch + a.v_offset + (size_t)head * a.vdim + c0 + c]));
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * LA_CHUNK; e += LA_THREADS) {
      const int t = e / LA_CHUNK, j = e - t * LA_CHUNK;
      float s = 0.f;
      if (j <= t) {
        const float* q = Q + t * qk_pitch;
        const float* k = K + j * qk_pitch;
        for (int d = 0; d < dim; ++d) s = fmaf(q[d], k[d], s);
        s *= power[t - j];
      }
      A[t * (LA_CHUNK + 1) + j] = s;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < n * vs; e += LA_THREADS) {
      const int t = e / vs, c = e - t * vs;
      float inside = 0.f, carried = 0.f;
      for (int j = 0; j <= t; ++j) inside = fmaf(A[t * (LA_CHUNK + 1) + j], V[j * a.slice_width + c], inside);
      const float* q = Q + t * qk_pitch;
      for (int d = 0; d < dim; ++d) carried = fmaf(q[d], S[d * a.slice_width + c], carried);
      a.out[(size_t)(row0 + t) * out_pitch + (size_t)head * a.vdim + c0 + c] = fmaf(power[t + 1], carried, inside);
    }
    __syncthreads();                                 // every read of the old state is done
    for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
      const int d = e / vs, c = e - d * vs;
      float add = 0.f;
      for (int j = 0; j < n; ++j) add = fmaf(power[n - 1 - j] * K[j * qk_pitch + d], V[j * a.slice_width + c], add);
      S[d * a.slice_width + c] = fmaf(power[n], S[d * a.slice_width + c], add);
    }
  }
  __syncthreads();
  if (a.read_only) return;
  for (int e = threadIdx.x; e < dim * vs; e += LA_THREADS) {
    const int d = e / vs, c = e - d * vs;
    state[(size_t)d * a.vdim + c] = S[d * a.slice_width + c];
  }
}

extern "C" int srb_lightning_scan(const void* proj, long long pitch, int q_offset, int k_offset, int v_offset,
                                  const int* cu_rows, const int* positions, const int* state_slots, float* state,
                                  const float* decay, float* out, int requests, int heads, int dim, int vdim,
                                  int read_only, int dtype, void* stream) {
  if (requests <= 0) return SRB_OK;
  if (heads <= 0 || dim <= 0 || vdim <= 0) SRB_FAIL("lightning_scan: heads, dim and vdim must be positive");
  if (requests > 65535) SRB_FAIL("lightning_scan: %d requests exceed one launch", requests);
  LightningArgs a;
  a.proj = proj; a.pitch = pitch; a.q_offset = q_offset; a.k_offset = k_offset; a.v_offset = v_offset;
  a.cu_rows = cu_rows; a.positions = positions; a.state_slots = state_slots; a.state = state; a.decay = decay; a.out = out;
  a.heads = heads; a.dim = dim; a.vdim = vdim; a.read_only = read_only;
  a.slices = (vdim + LA_SLICE - 1) / LA_SLICE;
  a.slice_width = (vdim + a.slices - 1) / a.slices;
  const size_t smem = ((size_t)dim * a.slice_width + 2 * (size_t)LA_CHUNK * (dim + 1) + (size_t)LA_CHUNK * a.slice_width +
                       (size_t)LA_CHUNK * (LA_CHUNK + 1) + LA_CHUNK + 1) * sizeof(float);
  if (smem > 220 * 1024) SRB_FAIL("lightning_scan: a state of %d x %d per head does not fit a block's shared memory", dim, vdim);
  dim3 grid(heads * a.slices, requests);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(lightning_scan_kernel<float>, grid, dim3(LA_THREADS), smem, s, a));
  } else if (dtype == SRB_DTYPE_BF16) {
    SRB_CUDA_CALL(cudaFuncSetAttribute(lightning_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    SRB_CUDA_CALL(srb_launch(lightning_scan_kernel<__nv_bfloat16>, grid, dim3(LA_THREADS), smem, s, a));
  } else {
    SRB_FAIL("lightning_scan: unknown dtype %d", dtype);
  }
  SRB_LAUNCH_CHECK("lightning_scan");
  return SRB_OK;
}

// One block per row: the heads' results are normed together, scaled, gated and rounded.
template <typename T>
__global__ void lightning_gate_norm_kernel(const float* __restrict__ o, const T* __restrict__ proj, long long pitch,
                                           int g_offset, const float* __restrict__ weight, float eps, int width,
                                           T* __restrict__ out) {
  __shared__ float reduce[33];
  srb_launch_dependents();
  srb_grid_dependency_wait();
  const int row = blockIdx.x;
  const float* src = o + (size_t)row * width;
  float squares = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) squares = fmaf(src[i], src[i], squares);
  const float inv = rsqrtf(srb_block_sum(squares, reduce) / (float)width + eps);
  const T* gate = proj + (size_t)row * pitch + g_offset;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float g = srb_to_float(gate[i]);
    out[(size_t)row * width + i] = srb_from_float<T>(src[i] * inv * weight[i] * (1.0f / (1.0f + expf(-g))));
  }
}

extern "C" int srb_lightning_gate_norm(const float* o, const void* proj, long long pitch, int g_offset, const float* weight,
                                       float eps, int rows, int width, void* out, int dtype, void* stream) {
  if (rows <= 0) return SRB_OK;
  if (width <= 0) SRB_FAIL("lightning_gate_norm: width %d must be positive", width);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SRB_DTYPE_F32)
    SRB_CUDA_CALL(srb_launch(lightning_gate_norm_kernel<float>, dim3(rows), dim3(256), 0, s, o, (const float*)proj, pitch,
                             g_offset, weight, eps, width, (float*)out));
  else if (dtype == SRB_DTYPE_BF16)
    SRB_CUDA_CALL(srb_launch(lightning_gate_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, s, o,
                             (const __nv_bfloat16*)proj, pitch, g_offset, weight, eps, width, (__nv_bfloat16*)out));
  else
    SRB_FAIL("lightning_gate_norm: unknown dtype %d", dtype);
  SRB_LAUNCH_CHECK("lightning_gate_norm");
  return SRB_OK;
}
