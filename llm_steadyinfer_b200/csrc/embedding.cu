// Embedding gather: out[t, :] = scale * table[tokens[t], :], widened to fp32 (the residual
// stream is fp32 in both precisions; the product with the scale is fp32 too). The reference's kernel
// (src/source/op/kernels/cuda/emb_kernel.cu:3-21) silently skips token ids outside
// the vocabulary; here such a row is zeroed and the status word is set.
#include "common.cuh"

template <typename TW>
__global__ void embedding_gather_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab,
                                        float scale, int* status) {
  pdl_prologue();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  float* o = out + (size_t)t * hidden;
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) set_status(status, SI_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* w = table + (size_t)tok * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = scale * to_f32<TW>(w[i]);
}

SI_EXPORT int si_embedding_gather(const int* tokens, const void* table, int table_dtype, float* out,
                                  int num_tokens, int hidden, int vocab, float scale, int* status,
                                  cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == SI_BF16)
    si_launch(embedding_gather_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream,
              tokens, (const __nv_bfloat16*)table, out, hidden, vocab, scale, status);
  else
    si_launch(embedding_gather_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream,
              tokens, (const float*)table, out, hidden, vocab, scale, status);
  return si_last_error();
}

// Embedding plus a hashed embedding of the token pair (previous, current):
//   out[t, :] = table[tok_t, :] + pair[r_t, :]
//   r_t = (tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets,  and r = buckets (the table's extra last row)
//   for the first token of a sequence.
// The previous token of a portion's first row is what the request's state slot holds (int32, one per slot);
// the block of that row reads it and then stores the portion's last token there for the next step, so the
// sequence may be cut anywhere and a token that was sampled on the device needs no trip to the host.
template <typename TW>
__global__ void embedding_pair_kernel(const int* __restrict__ tokens, const int* __restrict__ positions,
                                      const int* __restrict__ row_seq, const int* __restrict__ q_start,
                                      const int* __restrict__ slots, int* __restrict__ last_token,
                                      const TW* __restrict__ table, const TW* __restrict__ pair,
                                      float* __restrict__ out, int hidden, int vocab, int buckets,
                                      long long mul_prev, long long mul_cur, int num_seqs, int* status) {
  __shared__ int s_prev;
  pdl_prologue();
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const int seq = row_seq[t];
  float* o = out + (size_t)t * hidden;
  if (seq < 0 || seq >= num_seqs || tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0 && seq >= 0) set_status(status, seq >= num_seqs ? SI_BAD_SEQ : SI_BAD_TOKEN);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
    return;
  }
  if (threadIdx.x == 0) {
    const int row0 = q_start[seq];
    int prev;
    if (t > row0) {
      prev = tokens[t - 1];
    } else {
      int* slot = last_token + slots[seq];
      prev = *slot;
      *slot = tokens[q_start[seq + 1] - 1];           // what the next step's first row pairs with
    }
    s_prev = prev;
  }
  __syncthreads();
  long long r = buckets;
  if (positions[t] > 0) {
    const int prev = s_prev;
    if (prev < 0 || prev >= vocab) {
      if (threadIdx.x == 0) set_status(status, SI_BAD_TOKEN);
      for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = 0.f;
      return;
    }
    r = ((long long)prev * mul_prev + (long long)tok * mul_cur) % (long long)buckets;
  }
  const TW* w = table + (size_t)tok * hidden;
  const TW* b = pair + (size_t)r * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = to_f32<TW>(w[i]) + to_f32<TW>(b[i]);
}

SI_EXPORT int si_embedding_pair(const int* tokens, const int* positions, const int* row_seq, const int* q_start,
                                const int* slots, int* last_token, const void* table, const void* pair,
                                int table_dtype, float* out, int num_tokens, int hidden, int vocab, int buckets,
                                long long mul_prev, long long mul_cur, int num_seqs, int* status,
                                cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (buckets <= 0 || mul_prev < 0 || mul_cur < 0) return -2;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == SI_BF16)
    si_launch(embedding_pair_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, stream, tokens, positions,
              row_seq, q_start, slots, last_token, (const __nv_bfloat16*)table, (const __nv_bfloat16*)pair, out,
              hidden, vocab, buckets, mul_prev, mul_cur, num_seqs, status);
  else
    si_launch(embedding_pair_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, tokens, positions, row_seq,
              q_start, slots, last_token, (const float*)table, (const float*)pair, out, hidden, vocab, buckets,
              mul_prev, mul_cur, num_seqs, status);
  return si_last_error();
}
