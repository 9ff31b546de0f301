// Element-wise gated recurrences over the tokens of a step, with the state of every request in
// a slot of 32-bit floats that outlives the step.
//
// minGRU form (gates read the current token only):
//   z_t = sigmoid(a_t)            a = the gate's pre-activation (bias included)
//   c_t = u_t + 1/2 (u_t >= 0),  sigmoid(u_t) (u_t < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t
//   y_t = S_t * silu(g_t)
// a, u, g are the columns of one projection (float rows of a common stride); everything that
// enters the recurrence is 32-bit.  A request's tokens lie together (q_start[r] .. q_start[r+1]);
// its state is state[state_slots[r]][:], read at its first token and written back after its last.
//
// Two ways through a step.  Steps whose longest portion has at most CHUNK tokens: one launch, a
// thread a (request, channel), the tokens one after the other.  Longer portions: the recurrence
// S_out = A S_in + B of a piece of tokens composes, so a first launch reduces every piece of
// PIECE tokens to its (A, B) from a zero state, and a second launch starts every piece from
// the state that the pieces ahead of it compose to and writes the outputs; pieces run side by
// side.  The two ways differ in the rounding of the state only.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int SCAN_THREADS = 128;
constexpr int SCAN_CHUNK = 128;   // a step goes the chunked way when its longest portion exceeds this
constexpr int SCAN_PIECE = 32;    // tokens of one block of the chunked way (more blocks than with whole chunks)

__device__ __forceinline__ float sigmoid_f32(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float mingru_candidate(float u) { return u >= 0.0f ? u + 0.5f : sigmoid_f32(u); }

struct ScanArgs {
  const float* a;          // gate pre-activations   [T][in_stride]
  const float* u;          // candidate inputs
  const float* g;          // output gate inputs
  long long in_stride;
  void* y;                 // [T][y_stride], float or bfloat16
  long long y_stride;
  float* state;            // [n_slots][W]
  const int* q_start;      // [R+1]
  const int* state_slots;  // [R]
  int R, W, n_slots, n_chunks;
  float* ws_a;             // chunked way: [T / PIECE + R][W] each (see chunk_row), and [R][W] of incoming states
  float* ws_b;
  float* ws_s0;
  int* err;
};

// Where the piece that starts at token t0 of the step's r-th request keeps its (A, B): pieces of
// one request start PIECE tokens apart and a later request's tokens come later, so
// t0 / PIECE + r grows by at least one from any piece to the next and stays below T / PIECE + R.
__device__ __forceinline__ size_t chunk_row(int t0, int r) { return (size_t)(t0 / SCAN_PIECE + r); }

template <typename TO>
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_scan_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, ch = blockIdx.y * SCAN_THREADS + threadIdx.x;
  if (ch >= p.W) return;
  pdl_wait();
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const int slot = p.state_slots[r];
  if (t1 <= t0 || !sglc_index_ok(slot, p.n_slots, p.err)) return;
  float* sp = p.state + (size_t)slot * p.W + ch;
  float S = *sp;
  TO* y = reinterpret_cast<TO*>(p.y);
  for (int t = t0; t < t1; t += 4) {
    float a[4], u[4], g[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {             // a token's three loads do not wait for the token ahead
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      a[k] = on ? p.a[o] : 0.0f;
      u[k] = on ? p.u[o] : 0.0f;
      g[k] = on ? p.g[o] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      if (t + k < t1) {
        const float z = sigmoid_f32(a[k]);
        S = fmaf(z, mingru_candidate(u[k]), (1.0f - z) * S);
        y[(size_t)(t + k) * p.y_stride + ch] = from_f32<TO>(S * (g[k] * sigmoid_f32(g[k])));
      }
    }
  }
  *sp = S;
}

// chunk c of request r -> (A, B): S_out = A S_in + B
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_chunk_reduce_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, c = blockIdx.y, ch = blockIdx.z * SCAN_THREADS + threadIdx.x;
  if (ch >= p.W) return;
  pdl_wait();
  const int q0 = p.q_start[r], q1 = p.q_start[r + 1];
  const int t0 = q0 + c * SCAN_PIECE, t1 = min(t0 + SCAN_PIECE, q1);
  if (t0 >= q1) return;
  if (c == 0) {
    const int slot = p.state_slots[r];
    p.ws_s0[(size_t)r * p.W + ch] = sglc_index_ok(slot, p.n_slots, p.err) ? p.state[(size_t)slot * p.W + ch] : 0.0f;
  }
  float A = 1.0f, B = 0.0f;
  for (int t = t0; t < t1; t += 4) {
    float a[4], u[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      a[k] = on ? p.a[o] : 0.0f;
      u[k] = on ? p.u[o] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      if (t + k < t1) {
        const float z = sigmoid_f32(a[k]);
        A *= 1.0f - z;
        B = fmaf(z, mingru_candidate(u[k]), (1.0f - z) * B);
      }
    }
  }
  const size_t w = chunk_row(t0, r) * p.W + ch;
  p.ws_a[w] = A;
  p.ws_b[w] = B;
}

template <typename TO>
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_chunk_apply_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, c = blockIdx.y, ch = blockIdx.z * SCAN_THREADS + threadIdx.x;
  if (ch >= p.W) return;
  pdl_wait();
  const int q0 = p.q_start[r], q1 = p.q_start[r + 1];
  const int t0 = q0 + c * SCAN_PIECE, t1 = min(t0 + SCAN_PIECE, q1);
  if (t0 >= q1) return;
  float S = p.ws_s0[(size_t)r * p.W + ch];
  for (int k = 0; k < c; k++) {
    const size_t w = chunk_row(q0 + k * SCAN_PIECE, r) * p.W + ch;
    S = fmaf(p.ws_a[w], S, p.ws_b[w]);
  }
  TO* y = reinterpret_cast<TO*>(p.y);
  for (int t = t0; t < t1; t += 4) {
    float a[4], u[4], g[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      a[k] = on ? p.a[o] : 0.0f;
      u[k] = on ? p.u[o] : 0.0f;
      g[k] = on ? p.g[o] : 0.0f;
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      if (t + k < t1) {
        const float z = sigmoid_f32(a[k]);
        S = fmaf(z, mingru_candidate(u[k]), (1.0f - z) * S);
        y[(size_t)(t + k) * p.y_stride + ch] = from_f32<TO>(S * (g[k] * sigmoid_f32(g[k])));
      }
    }
  }
  if (t1 == q1) {
    const int slot = p.state_slots[r];
    if (sglc_index_ok(slot, p.n_slots, p.err)) p.state[(size_t)slot * p.W + ch] = S;
  }
}

SGLC_API int sglc_gated_scan_chunk() { return SCAN_CHUNK; }
SGLC_API int sglc_gated_scan_piece() { return SCAN_PIECE; }

// Floats of workspace the chunked way takes for a step of T tokens in R requests whose longest
// portion has max_q_len tokens (0: the step goes the one-launch way and needs none).
SGLC_API long long sglc_mingru_scan_workspace(int R, int W, int T, int max_q_len) {
  if (max_q_len <= SCAN_CHUNK) return 0;
  return (long long)W * (2LL * (T / SCAN_PIECE + R) + R);
}

// a, u, g: float, rows in_stride apart; y: [T][y_stride] of y_dtype; state: [n_slots][W] float;
// q_start: [R+1]; state_slots: [R]; T: tokens of the step; max_q_len: its longest portion; ws: the floats
// sglc_mingru_scan_workspace() names (may be null when that is 0).
SGLC_API int sglc_mingru_scan(const float* a, const float* u, const float* g, long long in_stride,
                              void* y, long long y_stride, int y_dtype, float* state, int n_slots,
                              const int* q_start, const int* state_slots, int R, int W, int T,
                              int max_q_len, float* ws, int* err, cudaStream_t stream) {
  if (R <= 0 || W <= 0) return SGLC_OK;
  if (y_dtype != SGLC_F32 && y_dtype != SGLC_BF16) return SGLC_ERR_ARGUMENT;
  ScanArgs p = {};
  p.a = a; p.u = u; p.g = g; p.in_stride = in_stride;
  p.y = y; p.y_stride = y_stride;
  p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.R = R; p.W = W; p.n_slots = n_slots; p.err = err;
  const int cb = (W + SCAN_THREADS - 1) / SCAN_THREADS;
  if (max_q_len <= SCAN_CHUNK) {
    if (cb > 65535) return SGLC_ERR_UNSUPPORTED;
    const dim3 grid(R, cb);
    if (y_dtype == SGLC_F32)
      return sglc_launch(mingru_scan_kernel<float>, grid, dim3(SCAN_THREADS), 0, stream, 1, true, p);
    return sglc_launch(mingru_scan_kernel<__nv_bfloat16>, grid, dim3(SCAN_THREADS), 0, stream, 1, true, p);
  }
  if (!ws) return SGLC_ERR_ARGUMENT;
  // (the grid depends on the longest portion in whole chunks only, as a captured graph's key does)
  p.n_chunks = (max_q_len + SCAN_CHUNK - 1) / SCAN_CHUNK * (SCAN_CHUNK / SCAN_PIECE);
  if (p.n_chunks > 65535 || cb > 65535) return SGLC_ERR_UNSUPPORTED;
  const size_t rows = (size_t)(T / SCAN_PIECE + R);
  p.ws_a = ws;
  p.ws_b = ws + rows * W;
  p.ws_s0 = ws + 2 * rows * W;
  const dim3 grid(R, p.n_chunks, cb);
  int rc = sglc_launch(mingru_chunk_reduce_kernel, grid, dim3(SCAN_THREADS), 0, stream, 1, true, p);
  if (rc != SGLC_OK) return rc;
  if (y_dtype == SGLC_F32)
    return sglc_launch(mingru_chunk_apply_kernel<float>, grid, dim3(SCAN_THREADS), 0, stream, 1, true, p);
  return sglc_launch(mingru_chunk_apply_kernel<__nv_bfloat16>, grid, dim3(SCAN_THREADS), 0, stream, 1, true, p);
}
