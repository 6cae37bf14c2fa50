// Retention over prompt portions in blocks of 64 tokens, float32 arithmetic on CUDA cores.
//
// The recurrence S_t = g S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (g: the head's decay) is linear with a constant decay, so
// a block of L <= 64 tokens that starts from the state S can be written without walking the tokens:
//     o_t = g^(t+1) S^T q_t + sum_{s <= t} g^(t-s) (k_s . q_t) v_s          (t, s count from the block's first token)
//     S'  = g^L S + sum_s g^(L-1-s) k_s v_s^T
// Four kernels:  rotate   q and k rotated by position, k scaled, float32 [T, H dk] each
//                delta    every block's own sum  sum_s g^(L-1-s) k_s v_s^T   (blocks side by side)
//                prefix   block after block: the state in front of each block (left where its sum was), the last one
//                         into the request's slot                             (the only sequential part: elementwise)
//                output   every block's o from its tokens and the state in front of it (blocks side by side)
// The token-by-token scan (recurrent.cu) keeps a token's state in registers and costs a chain of ~500 cycles a token;
// here a prompt's blocks run side by side.  The sums run in another order than the scan's (equal up to float32
// rounding), so the engine uses this form for the portions of the bfloat16 engine only: the 32-bit engine keeps the scan
// and with it the same bits for a prompt under every cut.
//
// A head's state lies column by column in its slot (element (i, j) at j * dk + i), as the scan keeps it.
#include "common.cuh"

#define RC_T 64            // tokens of a block
#define RC_N 128           // columns (or key rows) of a tile

// ---------------------------------------------------------------- rotate
// One block per row.  p [T, ld] float32: q heads at column 0 (H x dk), k at k_off.  The first `rot` elements of a head are
// rotated, element i paired with i + rot/2, angle = position * inv_freq[i]; k is multiplied by kscale afterwards.
__global__ void rc_rotate_kernel(const float* __restrict__ p, int ld, int k_off, const int* __restrict__ positions,
                                 const float* __restrict__ inv_freq, int rot, float kscale, float* __restrict__ Qr,
                                 float* __restrict__ Kr, int H, int dk) {
  const int row = blockIdx.x, half = rot >> 1, n = H * dk;
  const float pos = (float)positions[row];
  const float* pr = p + (size_t)row * ld;
  for (int idx = threadIdx.x; idx < n; idx += blockDim.x) {
    const int h = idx / dk, i = idx - h * dk;
    float q = pr[idx], k = pr[k_off + idx];
    if (i < rot) {
      const bool lo = i < half;
      const int partner = h * dk + (lo ? i + half : i - half);
      float sn, cs;
      sincosf(pos * inv_freq[lo ? i : i - half], &sn, &cs);
      const float qp = pr[partner], kp = pr[k_off + partner];
      q = lo ? q * cs - qp * sn : q * cs + qp * sn;
      k = lo ? k * cs - kp * sn : k * cs + kp * sn;
    }
    Qr[(size_t)row * n + idx] = q;
    Kr[(size_t)row * n + idx] = k * kscale;
  }
}

// powers of the decay by repeated multiplication (g^0 .. g^RC_T), as a token-by-token walk would form them
__device__ __forceinline__ void decay_powers(float* pw, float g) {
  if (threadIdx.x == 0) {
    float x = 1.f;
    for (int n = 0; n <= RC_T; ++n) { pw[n] = x; x *= g; }
  }
}

// ---------------------------------------------------------------- delta
// grid (blocks of the longest item, H * tiles of dk * tiles of dv, items), 256 threads = 16 x 16.
// dS[((item * max_blocks + c) * H + h)][j * dk + i] = sum_s g^(L-1-s) Kr[s][i] v[s][j]
__global__ void __launch_bounds__(256)
rc_delta_kernel(const float* __restrict__ Kr, const float* __restrict__ p, int ld, int v_off, const float* __restrict__ decay,
                const int* __restrict__ item_start, float* __restrict__ dS, int H, int dk, int dv, int max_blocks) {
  extern __shared__ __align__(16) float sm[];
  float* Kw = sm;                          // [RC_T][RC_N]
  float* Vs = Kw + RC_T * RC_N;            // [RC_T][RC_N]
  float* pw = Vs + RC_T * RC_N;            // [RC_T + 1]
  const int item = blockIdx.z, c = blockIdx.x;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  if (c * RC_T >= n) return;
  const int L = min(RC_T, n - c * RC_T), row0 = r0 + c * RC_T;
  const int it = (dk + RC_N - 1) / RC_N, jt = (dv + RC_N - 1) / RC_N;
  const int h = blockIdx.y / (it * jt), rem = blockIdx.y - h * (it * jt);
  const int i0 = (rem / jt) * RC_N, j0 = (rem % jt) * RC_N;
  decay_powers(pw, decay[h]);
  __syncthreads();
  for (int idx = threadIdx.x; idx < RC_T * RC_N; idx += 256) {
    const int s = idx / RC_N, x = idx - s * RC_N;
    const bool live = s < L;
    Kw[idx] = (live && i0 + x < dk) ? Kr[(size_t)(row0 + s) * (H * dk) + h * dk + i0 + x] * pw[L - 1 - s] : 0.f;
    Vs[idx] = (live && j0 + x < dv) ? p[(size_t)(row0 + s) * ld + v_off + h * dv + j0 + x] : 0.f;
  }
  __syncthreads();
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // i = i0 + tx + 16 u, j = j0 + ty + 16 w
  float acc[8][8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
#pragma unroll
    for (int w = 0; w < 8; ++w) acc[u][w] = 0.f;
  for (int s = 0; s < L; ++s) {
    float a[8], b[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = Kw[s * RC_N + tx + 16 * u];
#pragma unroll
    for (int w = 0; w < 8; ++w) b[w] = Vs[s * RC_N + ty + 16 * w];
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int w = 0; w < 8; ++w) acc[u][w] = fmaf(a[u], b[w], acc[u][w]);
  }
  float* out = dS + ((size_t)(item * max_blocks + c) * H + h) * ((size_t)dk * dv);
#pragma unroll
  for (int w = 0; w < 8; ++w) {
    const int j = j0 + ty + 16 * w;
    if (j >= dv) continue;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + tx + 16 * u;
      if (i < dk) out[(size_t)j * dk + i] = acc[u][w];
    }
  }
}

// ---------------------------------------------------------------- prefix
// grid (ceil(dk dv / 256), H, items).  Walks an item's blocks: leaves the state in front of block c where the block's
// own sum was, and the state behind the last block in the request's slot.
__global__ void __launch_bounds__(256)
rc_prefix_kernel(float* __restrict__ dS, float* __restrict__ state, long long slot_stride, const float* __restrict__ decay,
                 const int* __restrict__ item_start, const int* __restrict__ item_slot, int H, int dk, int dv, int max_blocks) {
  const int item = blockIdx.z, h = blockIdx.y;
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x, per = (size_t)dk * dv;
  if (e >= per) return;
  const int n = item_start[item + 1] - item_start[item];
  float* slot = state + (size_t)item_slot[item] * slot_stride + (size_t)h * per;
  const float g = decay[h];
  float gT = 1.f;
  for (int s = 0; s < RC_T; ++s) gT *= g;                       // g^64 by the same multiplications as the table's
  float S = slot[e];
  const int blocks = (n + RC_T - 1) / RC_T;
  float* cell0 = dS + ((size_t)item * max_blocks * H + h) * per + e;
  const size_t step = (size_t)H * per;
  // eight blocks' sums are asked for at once: only the multiply-adds form a chain
  for (int c0 = 0; c0 < blocks; c0 += 8) {
    float d[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) d[u] = c0 + u < blocks ? cell0[(size_t)(c0 + u) * step] : 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int c = c0 + u;
      if (c >= blocks) break;
      cell0[(size_t)c * step] = S;
      const int L = min(RC_T, n - c * RC_T);
      float gL = gT;
      if (L < RC_T) { gL = 1.f; for (int s = 0; s < L; ++s) gL *= g; }
      S = fmaf(gL, S, d[u]);
    }
  }
  slot[e] = S;
}

// ---------------------------------------------------------------- output
// grid (blocks of the longest item, H * tiles of dv, items), 256 threads = 16 x 16.
// o[t][j] = g^(t+1) sum_i Sb[i][j] Qr[t][i] + sum_{s <= t} g^(t-s) (Qr[t] . Kr[s]) v[s][j]
#define RC_KT 32           // key elements a step
__global__ void __launch_bounds__(256)
rc_output_kernel(const float* __restrict__ Qr, const float* __restrict__ Kr, const float* __restrict__ p, int ld, int v_off,
                 const float* __restrict__ Sb, const float* __restrict__ decay, const int* __restrict__ item_start,
                 float* __restrict__ out, int H, int dk, int dv, int max_blocks) {
  extern __shared__ __align__(16) float sm[];
  float* Qt = sm;                                  // [RC_T][RC_KT + 1]
  float* Kt = Qt + RC_T * (RC_KT + 1);             // [RC_T][RC_KT + 1]
  float* As = Kt + RC_T * (RC_KT + 1);             // [RC_T][RC_T + 1]
  float* Vs = As + RC_T * (RC_T + 1);              // [RC_T][RC_N]
  float* St = Vs + RC_T * RC_N;                    // [RC_KT][RC_N + 1]
  float* pw = St + RC_KT * (RC_N + 1);             // [RC_T + 1]
  const int item = blockIdx.z, c = blockIdx.x;
  const int r0 = item_start[item], n = item_start[item + 1] - r0;
  if (c * RC_T >= n) return;
  const int L = min(RC_T, n - c * RC_T), row0 = r0 + c * RC_T;
  const int jt = (dv + RC_N - 1) / RC_N;
  const int h = blockIdx.y / jt, j0 = (blockIdx.y - h * jt) * RC_N;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const size_t qk_ld = (size_t)H * dk;
  decay_powers(pw, decay[h]);
  for (int idx = threadIdx.x; idx < RC_T * RC_N; idx += 256) {
    const int s = idx / RC_N, x = idx - s * RC_N;
    Vs[idx] = (s < L && j0 + x < dv) ? p[(size_t)(row0 + s) * ld + v_off + h * dv + j0 + x] : 0.f;
  }
  // ---- A[t][s] = (Qr[t] . Kr[s]) g^(t-s) for s <= t: thread (ty, tx) owns t = ty + 16 a, s = tx + 16 b
  float a4[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) a4[a][b] = 0.f;
  for (int i0 = 0; i0 < dk; i0 += RC_KT) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < RC_T * RC_KT; idx += 256) {
      const int t = idx / RC_KT, x = idx - t * RC_KT;
      const bool live = t < L && i0 + x < dk;
      const size_t at = (size_t)(row0 + t) * qk_ld + h * dk + i0 + x;
      Qt[t * (RC_KT + 1) + x] = live ? Qr[at] : 0.f;
      Kt[t * (RC_KT + 1) + x] = live ? Kr[at] : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int x = 0; x < RC_KT; ++x) {
      float q[4], k[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) q[a] = Qt[(ty + 16 * a) * (RC_KT + 1) + x];
#pragma unroll
      for (int b = 0; b < 4; ++b) k[b] = Kt[(tx + 16 * b) * (RC_KT + 1) + x];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) a4[a][b] = fmaf(q[a], k[b], a4[a][b]);
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int t = ty + 16 * a, s = tx + 16 * b;
      As[t * (RC_T + 1) + s] = (s <= t && t < L) ? a4[a][b] * pw[t - s] : 0.f;
    }
  __syncthreads();
  // ---- o[t][j]: thread (ty, tx) owns t = ty + 16 a, j = j0 + tx + 16 w
  float intra[4][8], inter[4][8];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int w = 0; w < 8; ++w) intra[a][w] = inter[a][w] = 0.f;
  for (int s = 0; s < L; ++s) {
    float pa[4], v[8];
#pragma unroll
    for (int a = 0; a < 4; ++a) pa[a] = As[(ty + 16 * a) * (RC_T + 1) + s];
#pragma unroll
    for (int w = 0; w < 8; ++w) v[w] = Vs[s * RC_N + tx + 16 * w];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int w = 0; w < 8; ++w) intra[a][w] = fmaf(pa[a], v[w], intra[a][w]);
  }
  const float* Sh = Sb + ((size_t)(item * max_blocks + c) * H + h) * ((size_t)dk * dv);
  for (int i0 = 0; i0 < dk; i0 += RC_KT) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < RC_T * RC_KT; idx += 256) {
      const int t = idx / RC_KT, x = idx - t * RC_KT;
      Qt[t * (RC_KT + 1) + x] = (t < L && i0 + x < dk) ? Qr[(size_t)(row0 + t) * qk_ld + h * dk + i0 + x] : 0.f;
    }
    for (int idx = threadIdx.x; idx < RC_KT * RC_N; idx += 256) {
      const int jj = idx / RC_KT, x = idx - jj * RC_KT;               // consecutive threads: consecutive key rows of a column
      St[x * (RC_N + 1) + jj] = (i0 + x < dk && j0 + jj < dv) ? Sh[(size_t)(j0 + jj) * dk + i0 + x] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int x = 0; x < RC_KT; ++x) {
      float q[4], sv[8];
#pragma unroll
      for (int a = 0; a < 4; ++a) q[a] = Qt[(ty + 16 * a) * (RC_KT + 1) + x];
#pragma unroll
      for (int w = 0; w < 8; ++w) sv[w] = St[x * (RC_N + 1) + tx + 16 * w];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int w = 0; w < 8; ++w) inter[a][w] = fmaf(q[a], sv[w], inter[a][w]);
    }
  }
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int t = ty + 16 * a;
    if (t >= L) continue;
    const float gt = pw[t + 1];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int j = j0 + tx + 16 * w;
      if (j < dv) out[(size_t)(row0 + t) * ((size_t)H * dv) + h * dv + j] = fmaf(gt, inter[a][w], intra[a][w]);
    }
  }
}

// p float32 [T, ld]: q at column 0 (H x dk), k at k_off, v at v_off (H x dv).  scratch: float32, at least
// 2 * T * H * dk + n_items * max_blocks * H * dk * dv with max_blocks = ceil(max_item_rows / 64).  out float32 [T, H * dv].
FELLM_API int fellm_retention_chunked(const float* p, int ld, int k_off, int v_off, const int* positions,
                                      const float* inv_freq, int rot, const float* decay, float kscale, float* state,
                                      long long slot_stride, const int* item_start, const int* item_slot, float* out,
                                      float* scratch, int T, int n_items, int max_item_rows, int H, int dk, int dv,
                                      cudaStream_t stream) {
  if (n_items <= 0 || T <= 0) return 0;
  if (dk < 1 || dv < 1 || H < 1 || rot < 0 || rot > dk || (rot & 1) || max_item_rows < 1) return FELLM_ERR_SIZE;
  if (!p || !positions || !decay || !state || !item_start || !item_slot || !out || !scratch || (rot && !inv_freq)) return FELLM_ERR_ARG;
  const int max_blocks = (max_item_rows + RC_T - 1) / RC_T;
  float* Qr = scratch; float* Kr = Qr + (size_t)T * H * dk; float* dS = Kr + (size_t)T * H * dk;
  rc_rotate_kernel<<<T, 128, 0, stream>>>(p, ld, k_off, positions, inv_freq, rot, kscale, Qr, Kr, H, dk);
  const int it = (dk + RC_N - 1) / RC_N, jt = (dv + RC_N - 1) / RC_N;
  const size_t sm_delta = (size_t)(2 * RC_T * RC_N + RC_T + 1) * sizeof(float);
  const size_t sm_out = (size_t)(2 * RC_T * (RC_KT + 1) + RC_T * (RC_T + 1) + RC_T * RC_N + RC_KT * (RC_N + 1) + RC_T + 1) * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(rc_delta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_delta);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(rc_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_out);
  if (e != cudaSuccess) return (int)e;
  rc_delta_kernel<<<dim3(max_blocks, H * it * jt, n_items), 256, sm_delta, stream>>>(Kr, p, ld, v_off, decay, item_start, dS, H, dk, dv, max_blocks);
  const unsigned cells = (unsigned)(((size_t)dk * dv + 255) / 256);
  rc_prefix_kernel<<<dim3(cells, H, n_items), 256, 0, stream>>>(dS, state, slot_stride, decay, item_start, item_slot, H, dk, dv, max_blocks);
  rc_output_kernel<<<dim3(max_blocks, H * jt, n_items), 256, sm_out, stream>>>(Qr, Kr, p, ld, v_off, dS, decay, item_start, out, H, dk, dv, max_blocks);
  return launch_status();
}
