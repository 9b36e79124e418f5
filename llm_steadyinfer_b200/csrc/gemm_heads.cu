// One matrix per head, few rows: out[t, h, :] = a[t, h, :] @ w[h]^T for every head h in one launch, bf16 with fp32
// sums. a and out are rows with a head stride (views into wider rows are fine), w is [H, N, K]. For decode steps of
// mixers whose per-head matrices are too small for a launch each (the up-projections that latent attention moves to
// the query side and behind the attention). A warp owns an output column of a head: it streams the column's K
// weights once, 16 bytes a lane, against the rows staged in shared memory, and adds up over the lanes.
#include "common.cuh"

#define GH_MAX_ROWS 16
#define GH_WARPS 8

__global__ void __launch_bounds__(GH_WARPS * 32)
gemm_heads_kernel(const __nv_bfloat16* __restrict__ a, long long a_row, long long a_head,
                  const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out, long long o_row,
                  long long o_head, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char gh_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gh_smem);          // [M][K]
  pdl_prologue();
  const int h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kc = K / 8;
  for (int id = threadIdx.x; id < M * kc; id += blockDim.x) {
    const int m = id / kc, c = id % kc;
    reinterpret_cast<uint4*>(As)[id] = *reinterpret_cast<const uint4*>(a + (size_t)m * a_row + (size_t)h * a_head + c * 8);
  }
  __syncthreads();
  const int n = blockIdx.x * GH_WARPS + warp;
  if (n >= N) return;
  const __nv_bfloat16* wr = w + ((size_t)h * N + n) * K;
  float acc[GH_MAX_ROWS];
#pragma unroll
  for (int m = 0; m < GH_MAX_ROWS; ++m) acc[m] = 0.f;
  for (int c = lane; c < kc; c += 32) {
    const uint4 wv = *reinterpret_cast<const uint4*>(wr + c * 8);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
    float wf[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(w2[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
    for (int m = 0; m < GH_MAX_ROWS; ++m) {
      if (m >= M) break;
      const uint4 av = reinterpret_cast<const uint4*>(As)[m * kc + c];
      const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(a2[i]);
        acc[m] = fmaf(f.x, wf[2 * i], acc[m]);
        acc[m] = fmaf(f.y, wf[2 * i + 1], acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < GH_MAX_ROWS; ++m) {
    if (m >= M) break;
    const float v = warp_sum(acc[m]);
    if (lane == 0) out[(size_t)m * o_row + (size_t)h * o_head + n] = __float2bfloat16_rn(v);
  }
}

SI_EXPORT int si_gemm_heads(const void* a, long long a_row, long long a_head, const void* w, void* out, long long o_row,
                            long long o_head, int M, int H, int N, int K, cudaStream_t stream) {
  if (M <= 0 || H <= 0 || N <= 0) return 0;
  if (M > GH_MAX_ROWS || K % 8 || K <= 0 || H > 65535) return -2;
  const size_t smem = (size_t)M * K * sizeof(__nv_bfloat16);
  if (smem > 48 * 1024) return -2;
  si_launch(gemm_heads_kernel, dim3((N + GH_WARPS - 1) / GH_WARPS, H), dim3(GH_WARPS * 32), smem, stream,
            (const __nv_bfloat16*)a, a_row, a_head, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row, o_head, M, N, K);
  return si_last_error();
}
