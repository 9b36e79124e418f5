// Kernels of the state-space mixer (selective state space with a scalar decay per head) and of the short causal
// convolution in front of it. Everything that enters the recurrence is fp32: the step size, the decay, the state
// and the sums; the inputs are the projection's output in the compute dtype.
//
// Per request the mixer keeps one fp32 vector in its state slot:
//   [ recurrent state: heads * Npad * P | the convolution's last K - 1 inputs: (K - 1) * C ]
// (Npad: N rounded up to what the scan's threads hold, si_ssm_padded_state; within a head the entries lie in the
// order of the scan's threads, so that a block reads and writes its state in whole lines)
// A portion of a sequence starts from what the slot holds (from zero when the portion starts at position 0) and
// leaves behind what the next portion needs, so a sequence may be cut anywhere.
//
//   conv:  y[t, c] = act(b[c] + sum_k w[c, k] * u[t - (K - 1) + k, c]),   u = 0 before the sequence
//   scan:  S_t = exp(-exp(a_log_h) * dt_t) * S_{t-1} + dt_t * B_t x_t^T   (S is N x P, per head h)
//          y_t = S_t^T C_t + D_h x_t,   dt_t = softplus(raw_t + dt_bias_h),   B, C of group h / (heads / groups)
//   gate:  g = y * silu(z);  out = g / sqrt(mean_part(g^2) + eps) * w     over `parts` equal parts of a row
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// ---- causal convolution + silu -------------------------------------------------------------------------------
// One thread per (row, channel). Inputs of earlier steps come from the slot's conv part [K - 1, C] (oldest
// first), those of this step from the rows before this one in the same portion.
template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ u, long long u_stride, const float* __restrict__ w,
                                   const float* __restrict__ b, const float* __restrict__ state,
                                   long long state_stride, long long conv_off, float* __restrict__ out,
                                   const int* __restrict__ positions, const int* __restrict__ row_seq,
                                   const int* __restrict__ q_start, const int* __restrict__ slots, int num_seqs,
                                   int C, int K, int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int seq = row_seq[t];
  if (seq < 0 || seq >= num_seqs) {
    if (seq >= 0 && threadIdx.x == 0) set_status(status, SI_BAD_SEQ);
    out[(size_t)t * C + c] = 0.f;
    return;
  }
  const int pos = positions[t];
  const int back = t - q_start[seq];                  // rows of this portion before this one
  const float* st = state + (size_t)slots[seq] * state_stride + conv_off;
  float acc = b[c];
  for (int k = 0; k < K; ++k) {
    const int j = K - 1 - k;                          // the input j tokens back
    float x;
    if (j > pos) x = 0.f;
    else if (j <= back) x = to_f32<T>(u[(size_t)(t - j) * u_stride + c]);
    else x = st[(size_t)(K - 1 - (j - back)) * C + c];    // j - back tokens before the portion
    acc = fmaf(w[(size_t)c * K + k], x, acc);
  }
  out[(size_t)t * C + c] = silu_f(acc);
}

// After the convolution of a step: the slot keeps the last K - 1 inputs of every sequence of the step.
// One thread per (sequence, channel); it reads what it needs of the old contents before it writes.
#define CONV_MAX_TAPS 16
template <typename T>
__global__ void conv_state_kernel(const T* __restrict__ u, long long u_stride, float* __restrict__ state,
                                  long long state_stride, long long conv_off, const int* __restrict__ q_start,
                                  const int* __restrict__ ctx_len, const int* __restrict__ slots, int C, int K) {
  pdl_prologue();
  const int s = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int row0 = q_start[s], n = q_start[s + 1] - row0;
  if (n <= 0) return;
  const int pos0 = ctx_len[s] - n;
  float* st = state + (size_t)slots[s] * state_stride + conv_off;
  float keep[CONV_MAX_TAPS];
  const int H = K - 1;
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    if (i >= H) break;
    // new entry i is the input at position pos0 + n - H + i
    const int r = n - H + i;                          // row within the portion, negative: before it
    float x;
    if (r >= 0) x = to_f32<T>(u[(size_t)(row0 + r) * u_stride + c]);
    else if (pos0 + r < 0) x = 0.f;
    else x = st[(size_t)(H + r) * C + c];
    keep[i] = x;
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    if (i >= H) break;
    st[(size_t)i * C + c] = keep[i];
  }
}

SI_EXPORT int si_causal_conv(const void* u, int dtype, long long u_stride, const float* w, const float* b,
                             float* state, long long state_stride, long long conv_off, float* out,
                             const int* positions, const int* row_seq, const int* q_start, const int* ctx_len,
                             const int* slots, int num_tokens, int num_seqs, int C, int K, int* status,
                             cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (K < 1 || K - 1 > CONV_MAX_TAPS || C > 65535 * 128 || num_seqs > 65535) return -2;
  const int threads = 128;
  dim3 grid(num_tokens, (C + threads - 1) / threads);
  dim3 sgrid((C + threads - 1) / threads, num_seqs);
  if (dtype == SI_BF16) {
    si_launch(causal_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)u, u_stride, w, b,
              (const float*)state, state_stride, conv_off, out, positions, row_seq, q_start, slots, num_seqs, C, K, status);
    if (K > 1)
      si_launch(conv_state_kernel<__nv_bfloat16>, sgrid, dim3(threads), 0, stream, (const __nv_bfloat16*)u, u_stride, state,
                state_stride, conv_off, q_start, ctx_len, slots, C, K);
  } else {
    si_launch(causal_conv_kernel<float>, grid, dim3(threads), 0, stream, (const float*)u, u_stride, w, b,
              (const float*)state, state_stride, conv_off, out, positions, row_seq, q_start, slots, num_seqs, C, K, status);
    if (K > 1)
      si_launch(conv_state_kernel<float>, sgrid, dim3(threads), 0, stream, (const float*)u, u_stride, state,
                state_stride, conv_off, q_start, ctx_len, slots, C, K);
  }
  return si_last_error();
}

// ---- the recurrence -------------------------------------------------------------------------------------------
// One block per (sequence of the step, head, cut of the columns). Thread (p, ns) keeps NPT entries of column p of
// the state in registers, in groups of four neighbouring n: entry i is S[((i / 4) * NS + ns) * 4 + i % 4, p], so that
// the NS threads of one p (neighbouring lanes) read B and C from shared memory as consecutive 16-byte words, without
// bank conflicts; they add their parts of y_t with shuffles. Tokens are walked in order, SCAN_CHUNK at a time; the
// chunk after the one being computed is on its way into the other half of shared memory meanwhile (cp.async for B,
// C and x; step size and decay by the first threads).
#define SCAN_CHUNK 32
#ifndef SCAN_UNROLL
#define SCAN_UNROLL 8        // tokens whose loads the compiler may issue ahead of the sums of the token before
#endif
constexpr int kScanUnroll = SCAN_UNROLL;

__device__ __forceinline__ void scan_cp16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}
__device__ __forceinline__ void scan_cp4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src));
}

template <typename T, int NPT>
__global__ void ssm_scan_kernel(const float* __restrict__ xbc, long long xbc_stride,     // conv output: [x | B | C]
                                const T* __restrict__ dt_raw, long long dt_stride,
                                const float* __restrict__ dt_bias, const float* __restrict__ a_log,
                                const float* __restrict__ Dskip, float* __restrict__ state, long long state_stride,
                                float* __restrict__ y, long long y_stride, const int* __restrict__ q_start,
                                const int* __restrict__ ctx_len, const int* __restrict__ slots, int heads,
                                int groups, int N, int P, int NS, int Pb) {
  extern __shared__ __align__(16) float sm[];
  pdl_prologue();
  const int s = blockIdx.x, h = blockIdx.y;
  const int row0 = q_start[s], n_rows = q_start[s + 1] - row0;
  if (n_rows <= 0) return;
  const int pos0 = ctx_len[s] - n_rows;
  const int g = h / (heads / groups);
  const int inner = heads * P;
  const int Npad = NS * NPT;
  const int Pbp = (Pb + 3) / 4 * 4;
  // two halves of [ B: CHUNK x Npad | C: CHUNK x Npad | x: CHUNK x Pbp | decay: CHUNK | step: CHUNK ]
  const int half_floats = 2 * SCAN_CHUNK * Npad + SCAN_CHUNK * Pbp + 2 * SCAN_CHUNK;
  const int tid = threadIdx.x;
  // the block's columns of the state: [p0, p0 + Pb) (blockIdx.z cuts P where that gives the device more blocks)
  const int p0 = blockIdx.z * Pb;
  const int ns = tid % NS;
  const bool live = tid / NS < Pb && p0 + tid / NS < P;      // threads beyond the columns follow idly
  const int p = live ? p0 + tid / NS : p0;
  const int gtid = p * NS + ns;            // the thread's place in the head's state, whatever the cut
  // the head's state in the order of the threads: entry i of thread gtid at i * (P * NS) + gtid
  float* st = state + (size_t)slots[s] * state_stride + (size_t)h * Npad * P;
  const int held = P * NS;
  float S[NPT];
#pragma unroll
  for (int i = 0; i < NPT; ++i) S[i] = (live && pos0 > 0) ? st[(size_t)i * held + gtid] : 0.f;
  const float rate = expf(a_log[h]);
  const float bias = dt_bias[h];
  const float dskip = Dskip[h];
  for (int idx = tid; idx < 2 * half_floats; idx += blockDim.x) sm[idx] = 0.f;      // the padding stays zero
  __syncthreads();
  // 16-byte copies where every source address is a multiple of 16 bytes
  const bool vec = (xbc_stride % 4 == 0) && (inner % 4 == 0) && (N % 4 == 0) && (P % 4 == 0) && (Pb % 4 == 0)
                   && ((size_t)xbc % 16 == 0);
  const int pcols = min(Pb, P - p0);

  auto stage = [&](int c0, int buf) {
    const int cn = min(SCAN_CHUNK, n_rows - c0);
    float* hB = sm + (size_t)buf * half_floats;
    float* hC = hB + SCAN_CHUNK * Npad;
    float* hX = hC + SCAN_CHUNK * Npad;
    float* hDec = hX + SCAN_CHUNK * Pbp;
    const float* base = xbc + (size_t)(row0 + c0) * xbc_stride;
    if (vec) {
      const int nq = N / 4, pq = pcols / 4;
      for (int idx = tid; idx < cn * nq; idx += blockDim.x) {
        const int r = idx / nq, q = idx % nq;
        const float* src = base + (size_t)r * xbc_stride + inner + (size_t)g * N + 4 * q;
        scan_cp16(hB + r * Npad + 4 * q, src);
        scan_cp16(hC + r * Npad + 4 * q, src + (size_t)groups * N);
      }
      for (int idx = tid; idx < cn * pq; idx += blockDim.x) {
        const int r = idx / pq, q = idx % pq;
        scan_cp16(hX + r * Pbp + 4 * q, base + (size_t)r * xbc_stride + (size_t)h * P + p0 + 4 * q);
      }
    } else {
      for (int idx = tid; idx < cn * N; idx += blockDim.x) {
        const int r = idx / N, n = idx % N;
        const float* src = base + (size_t)r * xbc_stride + inner + (size_t)g * N + n;
        scan_cp4(hB + r * Npad + n, src);
        scan_cp4(hC + r * Npad + n, src + (size_t)groups * N);
      }
      for (int idx = tid; idx < cn * pcols; idx += blockDim.x) {
        const int r = idx / pcols, pp = idx % pcols;
        scan_cp4(hX + r * Pbp + pp, base + (size_t)r * xbc_stride + (size_t)h * P + p0 + pp);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
    for (int idx = tid; idx < cn; idx += blockDim.x) {
      const float dt = softplus_f(to_f32<T>(dt_raw[(size_t)(row0 + c0 + idx) * dt_stride + h]) + bias);
      hDec[idx] = expf(-rate * dt);
      hDec[SCAN_CHUNK + idx] = dt;
    }
  };

  stage(0, 0);
  int buf = 0;
  for (int c0 = 0; c0 < n_rows; c0 += SCAN_CHUNK, buf ^= 1) {
    const int cn = min(SCAN_CHUNK, n_rows - c0);
    if (c0 + SCAN_CHUNK < n_rows) {
      stage(c0 + SCAN_CHUNK, buf ^ 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* hB = sm + (size_t)buf * half_floats;
    const float* hC = hB + SCAN_CHUNK * Npad;
    const float* hX = hC + SCAN_CHUNK * Npad;
    const float* hDec = hX + SCAN_CHUNK * Pbp;
    if (NS == 8) {
      // Eight lanes a column: the lanes' partial sums of eight tokens are added up together by exchanging halves
      // (4 + 2 + 1 shuffles for eight tokens, and off the per-token chain), lane ns ending with token ns of the eight.
      for (int r0 = 0; r0 < cn; r0 += 8) {
        float acc[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc[u] = 0.f;
          if (r0 + u < cn) {
            const int r = r0 + u;
            const float dec = hDec[r];
            const float dx = hX[r * Pbp + p - p0] * hDec[SCAN_CHUNK + r];
            const float4* Br = reinterpret_cast<const float4*>(hB + r * Npad) + ns;
            const float4* Cr = reinterpret_cast<const float4*>(hC + r * Npad) + ns;
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int i4 = 0; i4 < NPT / 4; ++i4) {
              const float4 b = Br[i4 * 8], c = Cr[i4 * 8];
              S[4 * i4 + 0] = fmaf(dec, S[4 * i4 + 0], dx * b.x); a0 = fmaf(S[4 * i4 + 0], c.x, a0);
              S[4 * i4 + 1] = fmaf(dec, S[4 * i4 + 1], dx * b.y); a1 = fmaf(S[4 * i4 + 1], c.y, a1);
              S[4 * i4 + 2] = fmaf(dec, S[4 * i4 + 2], dx * b.z); a0 = fmaf(S[4 * i4 + 2], c.z, a0);
              S[4 * i4 + 3] = fmaf(dec, S[4 * i4 + 3], dx * b.w); a1 = fmaf(S[4 * i4 + 3], c.w, a1);
            }
            acc[u] = a0 + a1;
          }
        }
        const bool b4 = ns & 4, b2 = ns & 2, b1 = ns & 1;
        float h4[4], h2[2];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          h4[u] = (b4 ? acc[4 + u] : acc[u]) + __shfl_xor_sync(0xffffffffu, b4 ? acc[u] : acc[4 + u], 4);
#pragma unroll
        for (int u = 0; u < 2; ++u)
          h2[u] = (b2 ? h4[2 + u] : h4[u]) + __shfl_xor_sync(0xffffffffu, b2 ? h4[u] : h4[2 + u], 2);
        const float v = (b1 ? h2[1] : h2[0]) + __shfl_xor_sync(0xffffffffu, b1 ? h2[0] : h2[1], 1);
        const int r = r0 + ns;
        if (r < cn && live) y[(size_t)(row0 + c0 + r) * y_stride + (size_t)h * P + p] = v + dskip * hX[r * Pbp + p - p0];
      }
    } else {
#pragma unroll kScanUnroll
    for (int r = 0; r < cn; ++r) {
      const float dec = hDec[r];
      const float xr = hX[r * Pbp + p - p0];
      const float dx = xr * hDec[SCAN_CHUNK + r];
      const float4* Br = reinterpret_cast<const float4*>(hB + r * Npad) + ns;
      const float4* Cr = reinterpret_cast<const float4*>(hC + r * Npad) + ns;
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < NPT / 4; ++i4) {
        const float4 b = Br[i4 * NS], c = Cr[i4 * NS];
        S[4 * i4 + 0] = fmaf(dec, S[4 * i4 + 0], dx * b.x); acc0 = fmaf(S[4 * i4 + 0], c.x, acc0);
        S[4 * i4 + 1] = fmaf(dec, S[4 * i4 + 1], dx * b.y); acc1 = fmaf(S[4 * i4 + 1], c.y, acc1);
        S[4 * i4 + 2] = fmaf(dec, S[4 * i4 + 2], dx * b.z); acc0 = fmaf(S[4 * i4 + 2], c.z, acc0);
        S[4 * i4 + 3] = fmaf(dec, S[4 * i4 + 3], dx * b.w); acc1 = fmaf(S[4 * i4 + 3], c.w, acc1);
      }
      float acc = acc0 + acc1;
      for (int o = NS >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o, NS);
      if (ns == 0 && live) y[(size_t)(row0 + c0 + r) * y_stride + (size_t)h * P + p] = acc + dskip * xr;
    }
    }
    __syncthreads();       // everyone is done with this half before it is filled again
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) st[(size_t)i * held + gtid] = S[i];
  }
}

template <typename T, int NPT>
static int scan_launch(const float* xbc, long long xbc_stride, const void* dt_raw, long long dt_stride,
                       const float* dt_bias, const float* a_log, const float* Dskip, float* state,
                       long long state_stride, float* y, long long y_stride, const int* q_start, const int* ctx_len,
                       const int* slots, int num_seqs, int heads, int groups, int N, int P, int NS, cudaStream_t stream) {
  // Cut the columns over more blocks while the blocks still find a multiprocessor each, down to 8 columns a block:
  // a block's time goes to reading B and C from shared memory once per column, so columns on idle multiprocessors
  // are time saved; beyond one block each, the cut only repeats the staging of B and C (measured at 64 heads, one
  // sequence of 2,048 rows: 128 blocks 0.63 ms, 256 blocks 0.74 ms, 512 blocks of 8 columns 1.35 ms). The state's
  // layout does not depend on the cut.
  int Pb = P;
  while (Pb % 2 == 0 && Pb / 2 >= 8 && 2LL * num_seqs * heads * (P / Pb) <= si_sm_count()) Pb /= 2;
  int threads = (Pb * NS + 31) / 32 * 32;
  const size_t smem = (size_t)2 * (2 * SCAN_CHUNK * NS * NPT + SCAN_CHUNK * ((Pb + 3) / 4 * 4) + 2 * SCAN_CHUNK) * sizeof(float);
  if (smem > 200 * 1024) return -2;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(ssm_scan_kernel<T, NPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -2;
  }
  si_launch(ssm_scan_kernel<T, NPT>, dim3(num_seqs, heads, P / Pb), dim3(threads), smem, stream, xbc, xbc_stride,
            (const T*)dt_raw, dt_stride, dt_bias, a_log, Dskip, state, state_stride, y, y_stride, q_start, ctx_len,
            slots, heads, groups, N, P, NS, Pb);
  return si_last_error();
}

// How the scan spreads a head's N x P state over its threads: NS lanes per column (a power of two up to 32), each
// with NPT entries (4, 8, 16 or 32). Returns NS and sets *npt; N is padded to NS * NPT.
static int scan_shape(int N, int P, int* npt) {
  int NS = 32;
  while (NS > 1 && (P * NS > 1024 || NS * 2 > N)) NS >>= 1;
  while (NS > 1 && P * NS > 512 && (N + NS / 2 - 1) / (NS / 2) <= 16) NS >>= 1;     // fewer, fuller threads
  while (NS > 1 && (N + NS - 1) / NS < 4) NS >>= 1;                                  // at least four entries each
  const int per = (N + NS - 1) / NS;
  *npt = per <= 4 ? 4 : per <= 8 ? 8 : per <= 16 ? 16 : 32;
  return per > 32 ? 0 : NS;
}

// N rounded up to the state rows the scan keeps per head (the state tensor holds heads * this * P floats).
SI_EXPORT int si_ssm_padded_state(int N, int P) {
  int npt = 0;
  const int NS = scan_shape(N, P, &npt);
  return NS * npt;
}

SI_EXPORT int si_ssm_scan(const float* xbc, long long xbc_stride, const void* dt_raw, int dtype, long long dt_stride,
                          const float* dt_bias, const float* a_log, const float* Dskip, float* state,
                          long long state_stride, float* y, long long y_stride, const int* q_start,
                          const int* ctx_len, const int* slots, int num_seqs, int heads, int groups, int N, int P,
                          cudaStream_t stream) {
  if (num_seqs <= 0) return 0;
  if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || P <= 0 || P > 1024 || heads > 65535) return -2;
  int per = 0;
  const int NS = scan_shape(N, P, &per);
  if (NS == 0) return -2;
#define SCAN_GO(TT, NPT) scan_launch<TT, NPT>(xbc, xbc_stride, dt_raw, dt_stride, dt_bias, a_log, Dskip, state, \
                                              state_stride, y, y_stride, q_start, ctx_len, slots, num_seqs, heads, \
                                              groups, N, P, NS, stream)
  if (dtype == SI_BF16) {
    if (per <= 4) return SCAN_GO(__nv_bfloat16, 4);
    if (per <= 8) return SCAN_GO(__nv_bfloat16, 8);
    if (per <= 16) return SCAN_GO(__nv_bfloat16, 16);
    return SCAN_GO(__nv_bfloat16, 32);
  }
  if (per <= 4) return SCAN_GO(float, 4);
  if (per <= 8) return SCAN_GO(float, 8);
  if (per <= 16) return SCAN_GO(float, 16);
  return SCAN_GO(float, 32);
#undef SCAN_GO
}

// ---- gate and norm in parts -----------------------------------------------------------------------------------
// One block per (row, part): g = y * silu(z); out = g / sqrt(mean(g^2) + eps) * w.
template <typename T>
__global__ void gated_part_norm_kernel(const float* __restrict__ y, long long y_stride, const T* __restrict__ z,
                                       long long z_stride, const float* __restrict__ w, T* __restrict__ out,
                                       long long out_stride, int part, float eps) {
  __shared__ float red[33];
  pdl_prologue();
  const int t = blockIdx.x, c0 = blockIdx.y * part;
  const float* yr = y + (size_t)t * y_stride + c0;
  const T* zr = z + (size_t)t * z_stride + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float g = yr[i] * silu_f(to_f32<T>(zr[i]));
    ss += g * g;
  }
  ss = block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)part + eps);
  T* o = out + (size_t)t * out_stride + c0;
  for (int i = threadIdx.x; i < part; i += blockDim.x) {
    const float g = yr[i] * silu_f(to_f32<T>(zr[i]));
    o[i] = from_f32<T>(g * rs * w[c0 + i]);
  }
}

SI_EXPORT int si_gated_part_norm(const float* y, long long y_stride, const void* z, int dtype, long long z_stride,
                                 const float* w, void* out, long long out_stride, int rows, int width, int parts,
                                 float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (parts <= 0 || width % parts || parts > 65535) return -2;
  const int part = width / parts;
  const int threads = part >= 512 ? 256 : 128;
  if (dtype == SI_BF16)
    si_launch(gated_part_norm_kernel<__nv_bfloat16>, dim3(rows, parts), dim3(threads), 0, stream, y, y_stride,
              (const __nv_bfloat16*)z, z_stride, w, (__nv_bfloat16*)out, out_stride, part, eps);
  else
    si_launch(gated_part_norm_kernel<float>, dim3(rows, parts), dim3(threads), 0, stream, y, y_stride,
              (const float*)z, z_stride, w, (float*)out, out_stride, part, eps);
  return si_last_error();
}
