// A short causal convolution over time per channel, with what follows it in a recurrent mixer's
// input path, for the tokens of a step:
//   c_t[ch] = sum_{j < K} taps[ch][j] * x_{t-(K-1)+j}[ch]     (the last tap is the current token's)
//   y_t[ch] = silu(c_t[ch])
// and, for the segments that ask for it, each head's row made a unit vector and scaled:
//   y <- y / sqrt(sum(y^2) + unit_eps) * scale.
// x before a request's first token is zero.  A request's last K-1 inputs are part of its state:
// tail[slot][m][ch], m = 0 the oldest; a portion reads the tail where it reaches back before its
// own first token, and a second kernel moves the tail on behind it (it waits for the first to
// end: nothing reads a tail that is being rewritten).  In a step of single tokens (every request
// brings one) a channel's tail has one reader, the thread that computes the channel, which then
// moves it on itself: one launch.  Everything is 32-bit.
//
// The same launch makes the per-head gates of a gated delta rule from two more columns blocks of x:
//   beta = sigmoid(x_b),   decay = exp(-exp(A_log) * softplus(x_a + dt_bias)).
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int CONV_MAX_TAPS = 256;
constexpr int CONV_SEGS = 4;
constexpr int CONV_WARPS = 4;

struct ConvSeg {
  int col0;      // first channel of the segment (in x, taps, tail and y alike)
  int rows;      // head rows of the segment
  int width;     // channels of a row
  int unit;      // 1: the row becomes a unit vector times scale
  float scale;
};

struct ConvArgs {
  const float* x; long long x_stride;       // [T][x_stride]: projection results; channels are its first C columns
  const float* taps;                        // [C][K]
  float* tail;                              // [n_slots][K-1][C]
  float* y; long long y_stride;             // [T][C]
  const int* token_req;                     // [T]
  const int* q_start;                       // [R+1]
  const int* state_slots;                   // [R]
  int T, R, C, K, n_slots;
  float unit_eps;
  ConvSeg seg[CONV_SEGS];
  int n_seg, n_rows;
  int own_tail;                             // 1: every request brings one token; the kernel moves the tails on itself
  // gates (n_gate_heads = 0: none)
  int n_gate_heads, beta_col, a_col;
  const float* A_log; const float* dt_bias;
  float* gates; long long gates_stride;     // [T][2H]: beta, then decay
  int* err;
};

__device__ __forceinline__ float silu_f32(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f32(float v) { return fmaxf(v, 0.0f) + log1pf(expf(-fabsf(v))); }

constexpr int CONV_KEEP = 8;      // values of a row a lane keeps in registers (rows up to 256 wide; wider rows re-read y)

// A warp a head row: grid (tokens, groups of CONV_WARPS rows).  The last group's spare warps make the gates.
__global__ void __launch_bounds__(CONV_WARPS * 32)
short_conv_kernel(ConvArgs p) {
  pdl_launch_dependents();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.y * CONV_WARPS + warp;
  pdl_wait();
  const int r = p.token_req[t];
  const int q0 = p.q_start[r], i = t - q0;
  const int slot = p.state_slots[r];
  if (!sglc_index_ok(slot, p.n_slots, p.err)) return;
  const int K = p.K;
  if (row < p.n_rows) {
    float* tail = p.tail + (size_t)slot * (K - 1) * p.C;
    int s = 0, first = 0;
    while (s + 1 < p.n_seg && row >= first + p.seg[s].rows) { first += p.seg[s].rows; s++; }
    const ConvSeg sg = p.seg[s];
    const int c0 = sg.col0 + (row - first) * sg.width;
    float ss = 0.0f;
    float keep[CONV_KEEP];
#pragma unroll
    for (int n = 0; n < CONV_KEEP; n++) keep[n] = 0.0f;
    const bool kept = sg.width <= 32 * CONV_KEEP;
    for (int d = lane, n = 0; d < sg.width; d += 32, n++) {
      const int ch = c0 + d;
      float acc = 0.0f;
      for (int j = 0; j < K; j++) {
        const int src = i - (K - 1) + j;
        const float v = src >= 0 ? p.x[(size_t)(q0 + src) * p.x_stride + ch] : tail[(size_t)(K - 1 + src) * p.C + ch];
        acc = fmaf(p.taps[(size_t)ch * K + j], v, acc);
      }
      const float a = silu_f32(acc);
      ss = fmaf(a, a, ss);
      if (kept) {
#pragma unroll
        for (int m = 0; m < CONV_KEEP; m++)
          if (m == n) keep[m] = a;
      }
      if (!kept || !sg.unit) p.y[(size_t)t * p.y_stride + ch] = a;
      if (p.own_tail && K > 1) {               // (ascending: an entry is read before its place is written)
        for (int m = 0; m + 1 < K - 1; m++) tail[(size_t)m * p.C + ch] = tail[(size_t)(m + 1) * p.C + ch];
        tail[(size_t)(K - 2) * p.C + ch] = p.x[(size_t)t * p.x_stride + ch];
      }
    }
    if (sg.unit) {
      ss = warp_sum(ss);
      const float f = sg.scale / sqrtf(ss + p.unit_eps);
      if (kept) {
#pragma unroll
        for (int m = 0; m < CONV_KEEP; m++) {
          const int d = lane + 32 * m;
          if (d < sg.width) p.y[(size_t)t * p.y_stride + c0 + d] = keep[m] * f;
        }
      } else {
        __syncwarp();
        for (int d = lane; d < sg.width; d += 32) p.y[(size_t)t * p.y_stride + c0 + d] *= f;
      }
    }
  } else if (blockIdx.y == gridDim.y - 1) {
    const int spare = (int)gridDim.y * CONV_WARPS - p.n_rows;          // warps of this block beyond the rows: at least one
    const int w = row - p.n_rows;
    for (int h = w * 32 + lane; h < p.n_gate_heads; h += spare * 32) {
      const float xb = p.x[(size_t)t * p.x_stride + p.beta_col + h];
      const float xa = p.x[(size_t)t * p.x_stride + p.a_col + h];
      p.gates[(size_t)t * p.gates_stride + h] = 1.0f / (1.0f + expf(-xb));
      p.gates[(size_t)t * p.gates_stride + p.n_gate_heads + h] = expf(-expf(p.A_log[h]) * softplus_f32(xa + p.dt_bias[h]));
    }
  }
}

// tail <- the last K-1 inputs of every request after this step's portion
__global__ void __launch_bounds__(128)
short_conv_tail_kernel(ConvArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, ch = blockIdx.y * 128 + threadIdx.x;
  pdl_wait();
  if (ch >= p.C) return;
  const int q0 = p.q_start[r], n = p.q_start[r + 1] - q0;
  const int slot = p.state_slots[r];
  if (n <= 0 || !sglc_index_ok(slot, p.n_slots, p.err)) return;
  const int K = p.K;
  float* tail = p.tail + (size_t)slot * (K - 1) * p.C;
  for (int m = 0; m < K - 1; m++) {            // ascending: an old entry is read before its place is written
    const int src = n - (K - 1) + m;
    tail[(size_t)m * p.C + ch] = src >= 0 ? p.x[(size_t)(q0 + src) * p.x_stride + ch] : tail[(size_t)(m + n) * p.C + ch];
  }
}

// segs: n_seg x {col0, rows, width, unit} as ints, scales: n_seg floats.
SGLC_API int sglc_short_conv(const float* x, long long x_stride, const float* taps, float* tail, float* y,
                             long long y_stride, const int* token_req, const int* q_start, const int* state_slots,
                             int T, int R, int C, int K, int n_slots, float unit_eps, const int* segs,
                             const float* scales, int n_seg, int n_gate_heads, int beta_col, int a_col,
                             const float* A_log, const float* dt_bias, float* gates, long long gates_stride,
                             int* err, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return SGLC_OK;
  if (K < 1 || K > CONV_MAX_TAPS || n_seg < 1 || n_seg > CONV_SEGS || C <= 0) return SGLC_ERR_UNSUPPORTED;
  ConvArgs p = {};
  p.x = x; p.x_stride = x_stride; p.taps = taps; p.tail = tail; p.y = y; p.y_stride = y_stride;
  p.token_req = token_req; p.q_start = q_start; p.state_slots = state_slots;
  p.T = T; p.R = R; p.C = C; p.K = K; p.n_slots = n_slots; p.unit_eps = unit_eps;
  p.n_seg = n_seg;
  for (int s = 0; s < n_seg; s++) {
    p.seg[s].col0 = segs[4 * s]; p.seg[s].rows = segs[4 * s + 1]; p.seg[s].width = segs[4 * s + 2];
    p.seg[s].unit = segs[4 * s + 3]; p.seg[s].scale = scales[s];
    p.n_rows += p.seg[s].rows;
  }
  p.n_gate_heads = n_gate_heads; p.beta_col = beta_col; p.a_col = a_col; p.A_log = A_log; p.dt_bias = dt_bias;
  p.gates = gates; p.gates_stride = gates_stride; p.err = err;
  p.own_tail = T == R ? 1 : 0;               // (R requests with at least a token each in T tokens: one each)
  // (one warp more than the rows when there are gates to make: the spare warps of the last group make them)
  const int groups = (p.n_rows + (n_gate_heads > 0 ? 1 : 0) + CONV_WARPS - 1) / CONV_WARPS;
  if (groups > 65535) return SGLC_ERR_UNSUPPORTED;
  int rc = sglc_launch(short_conv_kernel, dim3(T, groups), dim3(CONV_WARPS * 32), 0, stream, 1, true, p);
  if (rc != SGLC_OK || K == 1 || p.own_tail) return rc;
  return sglc_launch(short_conv_tail_kernel, dim3(R, (C + 127) / 128), dim3(128), 0, stream, 1, true, p);
}
