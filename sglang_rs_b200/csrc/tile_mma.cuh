// A 64 x 64 tile of C = A W^T on the tensor cores (bfloat16 in, 32-bit accumulation), for products whose rows
// are gathered or strided and whose weight matrix is chosen per tile (one matrix per expert, one per head):
// shapes that the plain products' kernels do not take.  mma.sync m16n8k16; 128 threads, warp (wy, wx) of a
// 2 x 2 grid owns 32 rows x 32 columns.  K is walked 32 at a time; the next step's operands travel from
// global memory into registers while the current step is multiplied from shared memory.
//
// The caller puts the address of every tile row of A into shared memory (null: the row does not exist and
// counts as zeros), so rows may come from anywhere.  NW weight matrices (1, or 2 for gate and up) share the
// A tile.  Every output element is accumulated over k in the same order whatever the tile holds, so a row's
// result does not depend on the rows beside it.
#pragma once
#include "common.cuh"
#include "mma_helpers.cuh"

#define TM_TILE 64
#define TM_K 32
#define TM_PITCH (TM_K + 8)       // 80-byte rows: the eight rows of an ldmatrix land in different banks

struct TileMmaSmem {
  __nv_bfloat16 a[TM_TILE][TM_PITCH];
  __nv_bfloat16 w[2][TM_TILE][TM_PITCH];
  const __nv_bfloat16* a_row[TM_TILE];
};

// eight consecutive values of a row, zeros behind `valid`; 16-byte loads where the address allows
__device__ __forceinline__ uint4 tm_load8(const __nv_bfloat16* p, int valid) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (!p || valid <= 0) return v;
  if (valid >= 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) return *reinterpret_cast<const uint4*>(p);
  __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
  for (int i = 0; i < 8 && i < valid; ++i) e[i] = p[i];
  return v;
}

// acc[w][i][j][4]: weight matrix w, m16 tile i (rows wy*32 + i*16 ..), n8 tile j (columns wx*32 + j*8 ..).
// w_base[m]: first row (output column) of the tile in matrix m, rows n_in apart; cols_valid columns exist.
template <int NW>
__device__ __forceinline__ void tile_mma_64x64(TileMmaSmem& s, const __nv_bfloat16* const (&w_base)[NW], int cols_valid,
                                               int n_in, float (&acc)[NW][2][4][4]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wy = warp >> 1, wx = warp & 1;
#pragma unroll
  for (int m = 0; m < NW; ++m)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][i][j][c] = 0.f;
  // a thread moves two 8-value pieces of A and of each W per step: piece p covers row p / 4, values (p % 4) * 8 ..
  uint4 ra[2], rw[NW][2];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int piece = tid + h * 128, row = piece >> 2, k = k0 + (piece & 3) * 8;
      const __nv_bfloat16* a = s.a_row[row];
      ra[h] = tm_load8(a ? a + k : nullptr, n_in - k);
#pragma unroll
      for (int m = 0; m < NW; ++m)
        rw[m][h] = tm_load8(row < cols_valid ? w_base[m] + (size_t)row * n_in + k : nullptr, n_in - k);
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int piece = tid + h * 128, row = piece >> 2, k = (piece & 3) * 8;
      *reinterpret_cast<uint4*>(&s.a[row][k]) = ra[h];
#pragma unroll
      for (int m = 0; m < NW; ++m) *reinterpret_cast<uint4*>(&s.w[m][row][k]) = rw[m][h];
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < n_in; k0 += TM_K) {
    __syncthreads();                     // the step before is multiplied
    stage();
    __syncthreads();
    if (k0 + TM_K < n_in) fetch(k0 + TM_K);
#pragma unroll
    for (int kk = 0; kk < TM_K; kk += 16) {
      unsigned a[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)
        ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3], &s.a[wy * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int m = 0; m < NW; ++m)
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          unsigned b0, b1, b2, b3;         // n8 tiles 2 jj and 2 jj + 1
          ldmatrix_x4(b0, b1, b2, b3, &s.w[m][wx * 32 + jj * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            mma_bf16(acc[m][i][2 * jj], a[i], b0, b1);
            mma_bf16(acc[m][i][2 * jj + 1], a[i], b2, b3);
          }
        }
    }
  }
}

// where element c of acc[..][i][j] lies in the tile
__device__ __forceinline__ int tile_mma_row(int i, int c) {
  return ((threadIdx.x >> 5) >> 1) * 32 + i * 16 + ((threadIdx.x & 31) >> 2) + (c >> 1) * 8;
}
__device__ __forceinline__ int tile_mma_col(int j, int c) {
  return ((threadIdx.x >> 5) & 1) * 32 + j * 8 + (threadIdx.x & 3) * 2 + (c & 1);
}

// ---- the same product on a 128 x 64 tile with asynchronous copies ----------------------------------------------
// For operands whose rows start on 16-byte boundaries (n_in a multiple of 8, aligned bases): 256 threads, warp (wy, wx)
// of a 4 x 2 grid owns 32 rows x 32 columns as above; K is walked 64 at a time through a ring of three stages that
// cp.async fills two steps ahead, so a block keeps two steps of operands in flight while it multiplies a third.  A
// tile of 128 rows reads each weight tile half as often as two tiles of 64 would.
#define TA_ROWS 128
#define TA_COLS 64
#define TA_STAGES 3
#define TA_K 64                    // a whole 128-byte line of every row per step
#define TA_PITCH (TA_K + 8)

// ROWS: rows of the A tile (128, or 32 for tiles that hold a few decoded tokens: the room that the smaller A buffer
// leaves goes into more stages, since such a tile has nothing to multiply and only streams its weights).
template <int NW, int ROWS = TA_ROWS, int STAGES = TA_STAGES> struct TileAsyncSmem {
  __nv_bfloat16 a[STAGES][ROWS][TA_PITCH];
  __nv_bfloat16 w[STAGES][NW][TA_COLS][TA_PITCH];
  const __nv_bfloat16* a_row[ROWS];
};

// rows_valid: rows of the tile that exist; a warp whose 16-row groups lie behind them multiplies nothing (with a few
// decoded tokens per expert most of the tile is empty, and the products of empty rows would cost more than the copies).
template <int NW, int ROWS = TA_ROWS, int STAGES = TA_STAGES>
__device__ __forceinline__ void tile_mma_128x64_async(TileAsyncSmem<NW, ROWS, STAGES>& s, const __nv_bfloat16* const (&w_base)[NW],
                                                      int cols_valid, int rows_valid, int n_in, float (&acc)[NW][2][4][4]) {
  constexpr int A_PIECES = ROWS * 8 / 256;                 // 16-byte pieces of A that a thread copies per step
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wy = warp >> 1, wx = warp & 1;
#pragma unroll
  for (int m = 0; m < NW; ++m)
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][i][j][c] = 0.f;
  const int steps = (n_in + TA_K - 1) / TA_K;
  // What a thread copies per step is fixed but for the step's offset along K: four 16-byte pieces of A (128 rows x 8
  // pieces) and two of each W (64 rows x 8 pieces).  Rows of A that do not exist are not copied at all: a row's result
  // depends on its own row only, and the results of such rows are never stored.
  const __nv_bfloat16* a_src[A_PIECES];
  const __nv_bfloat16* w_src[NW][2];
  int a_at[A_PIECES], w_at[2];
  const int k_of = (tid & 7) * 8;                          // the same for every piece of a thread (256 is a multiple of 8)
#pragma unroll
  for (int h = 0; h < A_PIECES; ++h) {
    const int row = (tid + h * 256) >> 3;
    a_at[h] = row * TA_PITCH + k_of;
    const __nv_bfloat16* a = row < rows_valid ? s.a_row[row] : nullptr;
    a_src[h] = a ? a + k_of : nullptr;
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = (tid + h * 256) >> 3;
    w_at[h] = row * TA_PITCH + k_of;
#pragma unroll
    for (int m = 0; m < NW; ++m) w_src[m][h] = row < cols_valid ? w_base[m] + (size_t)row * n_in + k_of : nullptr;
  }
  auto issue = [&](int step) {
    if (step < steps) {
      const int stage = step % STAGES, k0 = step * TA_K;
      const bool inside = k0 + k_of < n_in;
      __nv_bfloat16* a_stage = &s.a[stage][0][0];
#pragma unroll
      for (int h = 0; h < A_PIECES; ++h)
        if (a_src[h]) cp_async_16(a_stage + a_at[h], a_src[h] + k0, inside ? 16 : 0);
#pragma unroll
      for (int m = 0; m < NW; ++m) {
        __nv_bfloat16* w_stage = &s.w[stage][m][0][0];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const bool there = w_src[m][h] != nullptr && inside;
          cp_async_16(w_stage + w_at[h], there ? w_src[m][h] + k0 : w_base[0], there ? 16 : 0);
        }
      }
    }
    cp_async_commit();                                                    // an empty group keeps the count in step
  };
#pragma unroll
  for (int step = 0; step < STAGES - 1; ++step) issue(step);
  for (int step = 0; step < steps; ++step) {
    cp_async_wait<STAGES - 2>();                                       // the copies of this step have landed
    __syncthreads();                                                      // ... for every thread, and the step before is multiplied
    issue(step + STAGES - 1);                                             // into the stage that was multiplied last
    const int stage = step % STAGES;
    if (wy * 32 >= rows_valid || wy * 32 >= ROWS) continue;                                  // (the same for all lanes of the warp)
    const bool second = wy * 32 + 16 < rows_valid;
#pragma unroll
    for (int kk = 0; kk < TA_K; kk += 16) {
      unsigned a[2][4];
      ldmatrix_x4(a[0][0], a[0][1], a[0][2], a[0][3], &s.a[stage][wy * 32 + (lane & 15)][kk + (lane >> 4) * 8]);
      if (second) ldmatrix_x4(a[1][0], a[1][1], a[1][2], a[1][3], &s.a[stage][wy * 32 + 16 + (lane & 15)][kk + (lane >> 4) * 8]);
#pragma unroll
      for (int m = 0; m < NW; ++m)
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3,
                      &s.w[stage][m][wx * 32 + jj * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
          mma_bf16(acc[m][0][2 * jj], a[0], b0, b1);
          mma_bf16(acc[m][0][2 * jj + 1], a[0], b2, b3);
          if (second) {
            mma_bf16(acc[m][1][2 * jj], a[1], b0, b1);
            mma_bf16(acc[m][1][2 * jj + 1], a[1], b2, b3);
          }
        }
    }
  }
  cp_async_wait<0>();
}

// where element c of acc[..][i][j] lies in the 128 x 64 tile
__device__ __forceinline__ int tile_async_row(int i, int c) {
  return ((threadIdx.x >> 5) >> 1) * 32 + i * 16 + ((threadIdx.x & 31) >> 2) + (c >> 1) * 8;
}
__device__ __forceinline__ int tile_async_col(int j, int c) { return tile_mma_col(j, c); }
