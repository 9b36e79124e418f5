// The gated delta rule: a linear-attention recurrence whose state is a matrix per head that forgets by a scalar
// decay and is corrected, not just added to, by each token:
//   S <- g_t S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S is dk x dv, fp32
// so the read-out sees the token's own write. Everything that enters the recurrence is fp32.
//
// Two kernels. `delta_prepare` works on all rows at once: it makes q and k unit vectors per head
// (x / sqrt(sum(x^2) + 1e-6), q also times `q_scale`), beta = sigmoid(b) and g = exp(-exp(A_log) * softplus(a + dt_bias)).
// `delta_scan` walks the tokens of every sequence of the step in order. The columns of S are independent of one
// another, so a block takes (sequence, head, a cut of COLS columns); thread (column j, part p) keeps the rows
// p, p + NP, p + 2 NP, ... of column j in registers. Per token it forms its parts of k . S[:, j], q . S[:, j] and q . k
// from the old state, the NP parts of a column (neighbouring lanes) are added with shuffles, and then
//   kS = g (k . S_old[:, j]);  u_j = beta (v_j - kS);  o_j = g (q . S_old[:, j]) + (q . k) u_j;  S[:, j] <- g S_old[:, j] + k u_j
// which is the order above with one pass over the registers for the sums and one for the update. q, k, v, beta and g of
// CHUNK tokens are staged in shared memory at a time; within a chunk the warps do not wait for one another.
// A request's state is [heads, dk, dv] fp32 at the start of its slot; a portion that begins at position 0 starts from
// zero whatever the slot held.
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float softplus_d(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// xc: fp32 rows [q: G*dk | k: G*dk | ...] (the convolution's output), normalised in place.
// ba: rows of the projection holding b (H values at b_off) and a (H values at a_off) in the compute dtype.
// bg: fp32 [T, 2H]: beta, then g.
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(float* __restrict__ xc, long long xc_stride, const T* __restrict__ ba,
    long long ba_stride, int b_off, int a_off, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
    float* __restrict__ bg, int G, int H, int dk, float q_scale) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  float* row = xc + (size_t)t * xc_stride;
  for (int vec = warp; vec < 2 * G; vec += nwarps) {
    float* x = row + (size_t)vec * dk;
    float ss = 0.f;
    for (int i = lane; i < dk; i += 32) ss += x[i] * x[i];
    const float f = rsqrtf(warp_sum(ss) + 1e-6f) * (vec < G ? q_scale : 1.f);
    for (int i = lane; i < dk; i += 32) x[i] *= f;
  }
  const T* r = ba + (size_t)t * ba_stride;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    bg[(size_t)t * 2 * H + h] = 1.f / (1.f + expf(-to_f32<T>(r[b_off + h])));
    bg[(size_t)t * 2 * H + H + h] = expf(-expf(a_log[h]) * softplus_d(to_f32<T>(r[a_off + h]) + dt_bias[h]));
  }
}

SI_EXPORT int si_delta_prepare(float* xc, long long xc_stride, const void* ba, int dtype, long long ba_stride, int b_off,
                               int a_off, const float* a_log, const float* dt_bias, float* bg, int num_tokens, int G, int H,
                               int dk, float q_scale, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (dtype == SI_BF16)
    si_launch(delta_prepare_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(128), 0, stream, xc, xc_stride,
              (const __nv_bfloat16*)ba, ba_stride, b_off, a_off, a_log, dt_bias, bg, G, H, dk, q_scale);
  else
    si_launch(delta_prepare_kernel<float>, dim3(num_tokens), dim3(128), 0, stream, xc, xc_stride, (const float*)ba,
              ba_stride, b_off, a_off, a_log, dt_bias, bg, G, H, dk, q_scale);
  return si_last_error();
}

#define DELTA_CHUNK 16

// RPT: rows of a column that a thread keeps; NP = ceil(dk / RPT) rounded up to a power of two, at most 32.
template <int RPT>
__global__ void __launch_bounds__(256) delta_scan_kernel(const float* __restrict__ xc, long long xc_stride,
    const float* __restrict__ bg, float* __restrict__ state, long long state_stride, float* __restrict__ y,
    long long y_stride, const int* __restrict__ q_start, const int* __restrict__ ctx_len, const int* __restrict__ slots,
    int G, int H, int dk, int dv, int NP, int cols) {
  extern __shared__ float sm[];                 // [CHUNK][2 * dk + cols + 2]
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * cols;
  const int row0 = q_start[s], n = q_start[s + 1] - row0;
  if (n <= 0) return;
  const int pos0 = ctx_len[s] - n;
  const int g = h / (H / G);
  const int p = threadIdx.x % NP, jl = threadIdx.x / NP;
  const int j = j0 + jl;
  const bool col_ok = jl < cols && j < dv;
  float* S = state + (size_t)slots[s] * state_stride + (size_t)h * dk * dv;
  float st[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) {
    const int i = r * NP + p;
    st[r] = (col_ok && i < dk && pos0 > 0) ? S[(size_t)i * dv + j] : 0.f;
  }
  const int per_tok = 2 * dk + cols + 2;
  const size_t q_off = (size_t)g * dk, k_off = (size_t)(G + g) * dk, v_off = (size_t)2 * G * dk + (size_t)h * dv + j0;
  for (int c0 = 0; c0 < n; c0 += DELTA_CHUNK) {
    const int cn = min(DELTA_CHUNK, n - c0);
    __syncthreads();                            // the chunk before is done with
    for (int idx = threadIdx.x; idx < cn * per_tok; idx += blockDim.x) {
      const int tt = idx / per_tok, e = idx - tt * per_tok;
      const float* row = xc + (size_t)(row0 + c0 + tt) * xc_stride;
      float v;
      if (e < dk) v = row[q_off + e];
      else if (e < 2 * dk) v = row[k_off + e - dk];
      else if (e < 2 * dk + cols) v = (j0 + e - 2 * dk < dv) ? row[v_off + e - 2 * dk] : 0.f;
      else v = bg[(size_t)(row0 + c0 + tt) * 2 * H + (e - 2 * dk - cols) * H + h];      // beta, then g
      sm[idx] = v;
    }
    __syncthreads();
    for (int tt = 0; tt < cn; ++tt) {
      const float* qs = sm + (size_t)tt * per_tok;
      const float* ks = qs + dk;
      float sk = 0.f, sq = 0.f, qk = 0.f;
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int i = r * NP + p;
        const float kv = i < dk ? ks[i] : 0.f, qv = i < dk ? qs[i] : 0.f;
        sk = fmaf(kv, st[r], sk);
        sq = fmaf(qv, st[r], sq);
        qk = fmaf(qv, kv, qk);
      }
      for (int o = 1; o < NP; o <<= 1) {
        sk += __shfl_xor_sync(0xffffffffu, sk, o);
        sq += __shfl_xor_sync(0xffffffffu, sq, o);
        qk += __shfl_xor_sync(0xffffffffu, qk, o);
      }
      const float beta = qs[2 * dk + cols], gt = qs[2 * dk + cols + 1];
      const float vj = qs[2 * dk + (jl < cols ? jl : 0)];
      const float u = beta * (vj - gt * sk);
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int i = r * NP + p;
        const float kv = i < dk ? ks[i] : 0.f;
        st[r] = fmaf(kv, u, gt * st[r]);
      }
      if (p == 0 && col_ok) y[(size_t)(row0 + c0 + tt) * y_stride + (size_t)h * dv + j] = fmaf(qk, u, gt * sq);
    }
  }
  if (col_ok) {
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int i = r * NP + p;
      if (i < dk) S[(size_t)i * dv + j] = st[r];
    }
  }
}

// The launch shape for a state of dk x dv: rows a thread (RPT), parts a column (NP, a power of two up to 32),
// columns a block.
static void delta_shape(int dk, int dv, int* rpt, int* np, int* cols) {
  int r = 4;
  while (r < 64 && (dk + r - 1) / r > 32) r *= 2;       // at most 32 parts
  if (dk >= 64 && r < 8) r = 8;
  if (dk >= 128 && r < 16) r = 16;
  int parts = 1;
  while (parts * r < dk) parts *= 2;
  *rpt = r;
  *np = parts;
  int c = 256 / parts;
  if (c > dv) c = dv;
  if (c < 1) c = 1;
  *cols = c;
}

SI_EXPORT int si_delta_scan(const float* xc, long long xc_stride, const float* bg, float* state, long long state_stride,
                            float* y, long long y_stride, const int* q_start, const int* ctx_len, const int* slots,
                            int num_seqs, int G, int H, int dk, int dv, cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (G <= 0 || H % G || dk <= 0 || dv <= 0 || dk > 2048 || H > 65535) return -2;
  int rpt, np, cols;
  delta_shape(dk, dv, &rpt, &np, &cols);
  if (rpt * np < dk) return -2;
  const int zb = (dv + cols - 1) / cols;
  if (zb > 65535) return -2;
  const int threads = ((cols * np + 31) / 32) * 32;
  const size_t smem = (size_t)DELTA_CHUNK * (2 * dk + cols + 2) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  const dim3 grid(num_seqs, H, zb), block(threads);
#define DELTA_LAUNCH(R)                                                                                              \
  {                                                                                                                  \
    static size_t configured = 0;                                                                                    \
    if (smem > 48 * 1024 && smem > configured) {                                                                     \
      if (cudaFuncSetAttribute(delta_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return -2;                                                                                                   \
      configured = smem;                                                                                             \
    }                                                                                                                \
    si_launch(delta_scan_kernel<R>, grid, block, smem, stream, xc, xc_stride, bg, state, state_stride, y, y_stride,  \
              q_start, ctx_len, slots, G, H, dk, dv, np, cols);                                                      \
  }
  if (rpt == 4) DELTA_LAUNCH(4)
  else if (rpt == 8) DELTA_LAUNCH(8)
  else if (rpt == 16) DELTA_LAUNCH(16)
  else if (rpt == 32) DELTA_LAUNCH(32)
  else DELTA_LAUNCH(64)
#undef DELTA_LAUNCH
  return si_last_error();
}

// ---- the read-out's norm and gate ------------------------------------------------------------------------------------
//   out[t, h, :] = w * o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * silu(z[t, h, :])      w [dv] shared by the heads
// o fp32, z and out in the compute dtype (z a view with a row stride). One warp a (row, head).
template <typename T>
__global__ void __launch_bounds__(256) head_norm_gate_kernel(const float* __restrict__ o, long long o_stride, const T* __restrict__ z,
    long long z_stride, const float* __restrict__ w, T* __restrict__ out, long long out_stride, long long pairs, int H, int dv,
    float eps) {
  pdl_prologue();
  const long long wi = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (wi >= pairs) return;
  const int lane = threadIdx.x & 31;
  const long long t = wi / H;
  const int h = (int)(wi - t * H);
  const float* orow = o + t * o_stride + (size_t)h * dv;
  const T* zr = z + t * z_stride + (size_t)h * dv;
  float ss = 0.f;
  for (int i = lane; i < dv; i += 32) ss += orow[i] * orow[i];
  const float rs = rsqrtf(warp_sum(ss) / (float)dv + eps);
  T* dst = out + t * out_stride + (size_t)h * dv;
  for (int i = lane; i < dv; i += 32) {
    const float zz = to_f32<T>(zr[i]);
    dst[i] = from_f32<T>(orow[i] * rs * w[i] * (zz / (1.f + expf(-zz))));
  }
}

SI_EXPORT int si_head_norm_gate(const float* o, long long o_stride, const void* z, int dtype, long long z_stride,
                                const float* w, void* out, long long out_stride, int rows, int H, int dv, float eps,
                                cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (H <= 0 || dv <= 0) return -2;
  const long long pairs = (long long)rows * H;
  const dim3 grid((unsigned)((pairs + 7) / 8)), block(256);
  if (dtype == SI_BF16)
    si_launch(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, stream, o, o_stride, (const __nv_bfloat16*)z, z_stride, w,
              (__nv_bfloat16*)out, out_stride, pairs, H, dv, eps);
  else
    si_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, o_stride, (const float*)z, z_stride, w, (float*)out,
              out_stride, pairs, H, dv, eps);
  return si_last_error();
}
