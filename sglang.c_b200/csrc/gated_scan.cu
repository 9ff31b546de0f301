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

// V channels a thread (4: one 16-byte load per row and operand; a channel's own arithmetic is the
// same sequence either way, so its bits do not depend on V)
template <int V>
__device__ __forceinline__ void load_v(const float* p, bool on, float* out) {
  if (V == 4) {
    const float4 x = on ? *reinterpret_cast<const float4*>(p) : make_float4(0.f, 0.f, 0.f, 0.f);
    out[0] = x.x; out[1] = x.y; out[2] = x.z; out[3] = x.w;
  } else {
    out[0] = on ? *p : 0.0f;
  }
}
template <int V, typename TO>
__device__ __forceinline__ void store_y(TO* p, const float* v) {
  if (V == 4) {
    if constexpr (sizeof(TO) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]);
      *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1));
    }
  } else {
    p[0] = from_f32<TO>(v[0]);
  }
}
constexpr int SCAN_UNROLL = 8;    // tokens whose loads are in flight together
constexpr long long SCAN_VEC_MIN_THREADS = 148LL * 2048;

template <typename TO, int V>
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_scan_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, ch = (blockIdx.y * SCAN_THREADS + threadIdx.x) * V;
  if (ch >= p.W) return;
  pdl_wait();
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const int slot = p.state_slots[r];
  if (t1 <= t0 || !sglc_index_ok(slot, p.n_slots, p.err)) return;
  float* sp = p.state + (size_t)slot * p.W + ch;
  float S[V];
  load_v<V>(sp, true, S);
  TO* y = reinterpret_cast<TO*>(p.y);
  for (int t = t0; t < t1; t += SCAN_UNROLL) {
    float a[SCAN_UNROLL][V], u[SCAN_UNROLL][V], g[SCAN_UNROLL][V];
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {   // a token's three loads do not wait for the token ahead
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      load_v<V>(p.a + o, on, a[k]);
      load_v<V>(p.u + o, on, u[k]);
      load_v<V>(p.g + o, on, g[k]);
    }
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {
      if (t + k < t1) {
        float out[V];
#pragma unroll
        for (int c = 0; c < V; c++) {
          const float z = sigmoid_f32(a[k][c]);
          S[c] = fmaf(z, mingru_candidate(u[k][c]), (1.0f - z) * S[c]);
          out[c] = S[c] * (g[k][c] * sigmoid_f32(g[k][c]));
        }
        store_y<V, TO>(y + (size_t)(t + k) * p.y_stride + ch, out);
      }
    }
  }
  store_y<V, float>(sp, S);
}

// piece c of request r -> (A, B): S_out = A S_in + B
template <int V>
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_chunk_reduce_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, c = blockIdx.y, ch = (blockIdx.z * SCAN_THREADS + threadIdx.x) * V;
  if (ch >= p.W) return;
  pdl_wait();
  const int q0 = p.q_start[r], q1 = p.q_start[r + 1];
  const int t0 = q0 + c * SCAN_PIECE, t1 = min(t0 + SCAN_PIECE, q1);
  if (t0 >= q1) return;
  if (c == 0) {
    const int slot = p.state_slots[r];
    float s0[V];
    load_v<V>(p.state + (size_t)slot * p.W + ch, sglc_index_ok(slot, p.n_slots, p.err), s0);
    store_y<V, float>(p.ws_s0 + (size_t)r * p.W + ch, s0);
  }
  float A[V], B[V];
#pragma unroll
  for (int x = 0; x < V; x++) { A[x] = 1.0f; B[x] = 0.0f; }
  for (int t = t0; t < t1; t += SCAN_UNROLL) {
    float a[SCAN_UNROLL][V], u[SCAN_UNROLL][V];
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      load_v<V>(p.a + o, on, a[k]);
      load_v<V>(p.u + o, on, u[k]);
    }
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {
      if (t + k < t1) {
#pragma unroll
        for (int x = 0; x < V; x++) {
          const float z = sigmoid_f32(a[k][x]);
          A[x] *= 1.0f - z;
          B[x] = fmaf(z, mingru_candidate(u[k][x]), (1.0f - z) * B[x]);
        }
      }
    }
  }
  const size_t w = chunk_row(t0, r) * p.W + ch;
  store_y<V, float>(p.ws_a + w, A);
  store_y<V, float>(p.ws_b + w, B);
}

template <typename TO, int V>
__global__ void __launch_bounds__(SCAN_THREADS)
mingru_chunk_apply_kernel(ScanArgs p) {
  pdl_launch_dependents();
  const int r = blockIdx.x, c = blockIdx.y, ch = (blockIdx.z * SCAN_THREADS + threadIdx.x) * V;
  if (ch >= p.W) return;
  pdl_wait();
  const int q0 = p.q_start[r], q1 = p.q_start[r + 1];
  const int t0 = q0 + c * SCAN_PIECE, t1 = min(t0 + SCAN_PIECE, q1);
  if (t0 >= q1) return;
  float S[V];
  load_v<V>(p.ws_s0 + (size_t)r * p.W + ch, true, S);
  for (int k = 0; k < c; k++) {
    const size_t w = chunk_row(q0 + k * SCAN_PIECE, r) * p.W + ch;
    float A[V], B[V];
    load_v<V>(p.ws_a + w, true, A);
    load_v<V>(p.ws_b + w, true, B);
#pragma unroll
    for (int x = 0; x < V; x++) S[x] = fmaf(A[x], S[x], B[x]);
  }
  TO* y = reinterpret_cast<TO*>(p.y);
  for (int t = t0; t < t1; t += SCAN_UNROLL) {
    float a[SCAN_UNROLL][V], u[SCAN_UNROLL][V], g[SCAN_UNROLL][V];
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {
      const bool on = t + k < t1;
      const size_t o = (size_t)(t + k) * p.in_stride + ch;
      load_v<V>(p.a + o, on, a[k]);
      load_v<V>(p.u + o, on, u[k]);
      load_v<V>(p.g + o, on, g[k]);
    }
#pragma unroll
    for (int k = 0; k < SCAN_UNROLL; k++) {
      if (t + k < t1) {
        float out[V];
#pragma unroll
        for (int x = 0; x < V; x++) {
          const float z = sigmoid_f32(a[k][x]);
          S[x] = fmaf(z, mingru_candidate(u[k][x]), (1.0f - z) * S[x]);
          out[x] = S[x] * (g[k][x] * sigmoid_f32(g[k][x]));
        }
        store_y<V, TO>(y + (size_t)(t + k) * p.y_stride + ch, out);
      }
    }
  }
  if (t1 == q1) {
    const int slot = p.state_slots[r];
    if (sglc_index_ok(slot, p.n_slots, p.err)) store_y<V, float>(p.state + (size_t)slot * p.W + ch, S);
  }
}

// Tuning hook: -1 (default) lets the launcher choose how many channels a thread takes, 0 one, 1 four where legal.
static int g_scan_vec = -1;
SGLC_API void sglc_gated_scan_set_vec(int mode) { g_scan_vec = mode; }
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
  // four channels a thread where every row of every operand can be read 16 bytes at a time
  const bool legal4 = W % 4 == 0 && in_stride % 4 == 0 && y_stride % 4 == 0 &&
                      ((((uintptr_t)a | (uintptr_t)u | (uintptr_t)g | (uintptr_t)state | (uintptr_t)ws) & 15) == 0) &&
                      (((uintptr_t)y & (y_dtype == SGLC_F32 ? 15 : 7)) == 0);
  // ... and where a quarter of the threads still fills the machine (measured: 2,048 tokens of 768
  // channels 30 us a layer with one channel a thread, 63 us with four)
  const long long work = max_q_len <= SCAN_CHUNK ? (long long)R * W : (long long)(T / SCAN_PIECE + R) * W;
  const bool v4 = legal4 && (g_scan_vec == 1 || (g_scan_vec < 0 && work / 4 >= SCAN_VEC_MIN_THREADS));
  const int per_block = SCAN_THREADS * (v4 ? 4 : 1);
  const int cb = (W + per_block - 1) / per_block;
#define SCAN_LAUNCH(KERNEL, GRID)                                                                       \
  (v4 ? sglc_launch(KERNEL<4>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p)                          \
      : sglc_launch(KERNEL<1>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p))
#define SCAN_LAUNCH_T(KERNEL, GRID)                                                                     \
  (y_dtype == SGLC_F32                                                                                  \
       ? (v4 ? sglc_launch(KERNEL<float, 4>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p)            \
             : sglc_launch(KERNEL<float, 1>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p))           \
       : (v4 ? sglc_launch(KERNEL<__nv_bfloat16, 4>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p)    \
             : sglc_launch(KERNEL<__nv_bfloat16, 1>, GRID, dim3(SCAN_THREADS), 0, stream, 1, true, p)))
  if (max_q_len <= SCAN_CHUNK) {
    if (cb > 65535) return SGLC_ERR_UNSUPPORTED;
    const dim3 grid(R, cb);
    return SCAN_LAUNCH_T(mingru_scan_kernel, grid);
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
  int rc = SCAN_LAUNCH(mingru_chunk_reduce_kernel, grid);
  if (rc != SGLC_OK) return rc;
  return SCAN_LAUNCH_T(mingru_chunk_apply_kernel, grid);
#undef SCAN_LAUNCH
#undef SCAN_LAUNCH_T
}
