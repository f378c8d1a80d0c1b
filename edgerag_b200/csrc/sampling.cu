// Sampling over float logits: greedy argmax and temperature sampling by inverse CDF.
//
// One block per row.  A row with temperature <= 0 takes the first index of the maximum (the
// tie-break of an argmax that scans from the left).  Otherwise p = softmax(logits / T) in float
// and the token is the first index whose cumulative probability exceeds u, with u in [0, 1)
// derived from the row's 64-bit counter state by `uniform_from_state` below; the caller derives
// that state from (seed, request, index of the generated token), so a request's draws do not
// depend on what else is in the batch.
#include "common.cuh"

using namespace erb;

ERB_DEFINE_LAST_ERROR(erb_last_error)

namespace {

constexpr int kThreads = 256;

// splitmix64 finaliser; the top 24 bits give u = k / 2^24.
__host__ __device__ inline float uniform_from_state(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kThreads)
sample_rows_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                   const float* __restrict__ temperature, const long long* __restrict__ rng_state,
                   int* __restrict__ tokens) {
  chain_wait();
  __shared__ float s_val[32];
  __shared__ int s_idx[32];
  __shared__ float s_scan[kThreads];
  __shared__ int s_pick;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* x = logits + (size_t)row * row_stride;
  const float temp = temperature ? temperature[row] : 0.f;

  // Maximum and its first index.
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < vocab; i += kThreads) {
    const float v = x[i];
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if (lane == 0) { s_val[warp] = best; s_idx[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    best = lane < kThreads / 32 ? s_val[lane] : -INFINITY;
    best_i = lane < kThreads / 32 ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) { s_val[0] = best; s_idx[0] = best_i; }
  }
  __syncthreads();
  best = s_val[0];
  best_i = s_idx[0];
  if (!(temp > 0.f)) {
    if (tid == 0) tokens[row] = best_i == 0x7fffffff ? 0 : best_i;
    return;
  }

  // Each thread owns a contiguous chunk; chunk sums are scanned over the block in order.
  const float inv_t = 1.f / temp;
  const int chunk = (vocab + kThreads - 1) / kThreads;
  const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
  float local = 0.f;
  for (int i = lo; i < hi; ++i) local += expf((x[i] - best) * inv_t);
  s_scan[tid] = local;
  if (tid == 0) s_pick = vocab - 1;
  __syncthreads();
  if (tid == 0) {  // a serial scan of 256 values: fixed order, negligible time
    float run = 0.f;
    for (int j = 0; j < kThreads; ++j) { const float v = s_scan[j]; s_scan[j] = run; run += v; }
    s_val[1] = run;
  }
  __syncthreads();
  const float total = s_val[1];
  const float target = uniform_from_state((unsigned long long)rng_state[row]) * total;
  const float before = s_scan[tid];
  const float after = (tid + 1 < kThreads) ? s_scan[tid + 1] : total;
  if (local > 0.f && target >= before && target < after) {
    float run = before;
    int pick = hi - 1;
    for (int i = lo; i < hi; ++i) {
      run += expf((x[i] - best) * inv_t);
      if (run > target) { pick = i; break; }
    }
    s_pick = pick;  // exactly one thread's interval holds the target
  }
  __syncthreads();
  if (tid == 0) tokens[row] = s_pick;
}

}  // namespace

// logits: float [n_rows, row_stride]; temperature: float [n_rows] or null (all greedy);
// rng_state: int64 [n_rows] (ignored for greedy rows; may be null when temperature is null).
ERB_EXPORT int erb_sample_rows(const float* logits, long long row_stride, int n_rows, int vocab,
                               const float* temperature, const long long* rng_state, int* tokens,
                               void* stream) {
  if (n_rows <= 0) return ERB_OK;
  if (vocab <= 0 || row_stride < vocab) return fail(ERB_ERR_ARG, "sample_rows: bad vocab/stride");
  if (temperature && !rng_state) return fail(ERB_ERR_ARG, "sample_rows: temperature without rng_state");
  launch_chained(sample_rows_kernel, dim3(n_rows), dim3(kThreads), 0, (cudaStream_t)stream, logits, row_stride, vocab, temperature,
                                                                  rng_state, tokens);
  return check_launch("sample_rows");
}

// The uniform the kernel derives from a state, for callers that want to check a draw.
ERB_EXPORT float erb_uniform_from_state(long long state) {
  return uniform_from_state((unsigned long long)state);
}
