// Recurrences whose state is a matrix S [D x V] per head and request, in 32-bit floats that
// outlive the step (state[slot][head][D][V]), over the tokens of a step.
//
//   decay form (linear attention with a fixed decay per head):
//       S <- d_h S + k_t v_t^T                         o_t = S^T q_t
//   gated delta rule (per token a decay g_t and a step size b_t, both per head):
//       S <- g_t S;  u = b_t (v_t - S^T k_t);  S <- S + k_t u^T;   o_t = S^T q_t
// in this order: the read-out sees the current token's write.
//
// Column j of S needs nothing of the other columns: S^T k, the update and S^T q are, per column,
// two dot products and one scaled addition over D.  So a column belongs to L lanes of one warp that
// keep it in registers (32 entries each, D <= 32 L, entry e of lane s is row e L + s), a block
// takes a range of columns of one (request, head), and the tokens go by one after the other; the
// block stages the next tokens' q, k, v and gates in shared memory, eight at a time.
// q and k may have fewer heads than v (head h reads q/k head h / (H / G)).
// With `silu_in` the kernel applies silu to q, k and v as it stages them.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

constexpr int MS_PER = 32;        // entries of a column a lane keeps
constexpr int MS_BATCH = 8;       // tokens staged at a time
constexpr int MS_MAX_THREADS = 128;

enum { MS_DECAY = 0, MS_DELTA = 1 };

struct MsArgs {
  const float* q; long long q_stride;     // [T][..], head g at columns g*D
  const float* k; long long k_stride;
  const float* v; long long v_stride;     // head h at columns h*V
  const float* gates; long long gates_stride;   // delta: [T][2H] beta then decay
  const float* head_decay;                // decay form: [H]
  float* out; long long out_stride;       // [T][H*V]
  float* state;                           // [n_slots][H][D][V]
  const int* q_start; const int* state_slots;
  int R, H, G, D, V, n_slots, cols;       // cols: columns a block takes
  int silu_in;
  int* err;
};

__device__ __forceinline__ float ms_silu(float v) { return v / (1.0f + expf(-v)); }

template <int L, int MODE>
__global__ void __launch_bounds__(MS_MAX_THREADS)
matrix_state_kernel(MsArgs p) {
  constexpr int DP = MS_PER * L;
  extern __shared__ __align__(16) float sm[];
  float* ks = sm;                          // [BATCH][DP]
  float* qs = ks + MS_BATCH * DP;          // [BATCH][DP]
  float* vs = qs + MS_BATCH * DP;          // [BATCH][cols]
  float* gs = vs + MS_BATCH * p.cols;      // [BATCH][2]
  pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y, g = h / (p.H / p.G);
  const int tid = threadIdx.x, sub = tid % L, col = blockIdx.z * p.cols + tid / L;
  const bool on = tid / L < p.cols && col < p.V;
  pdl_wait();
  const int t0 = p.q_start[r], t1 = p.q_start[r + 1];
  const int slot = p.state_slots[r];
  if (t1 <= t0 || !sglc_index_ok(slot, p.n_slots, p.err)) return;
  float* sp = p.state + ((size_t)slot * p.H + h) * p.D * p.V;
  float S[MS_PER];
#pragma unroll
  for (int e = 0; e < MS_PER; e++) {
    const int i = e * L + sub;
    S[e] = (on && i < p.D) ? sp[(size_t)i * p.V + col] : 0.0f;
  }
  const float hd = MODE == MS_DECAY ? p.head_decay[h] : 0.0f;
  for (int tb = t0; tb < t1; tb += MS_BATCH) {
    const int nb = min(MS_BATCH, t1 - tb);
    __syncthreads();
    for (int x = tid; x < MS_BATCH * DP; x += blockDim.x) {
      const int b = x / DP, i = x % DP;
      float kv = 0.0f, qv = 0.0f;
      if (b < nb && i < p.D) {
        kv = p.k[(size_t)(tb + b) * p.k_stride + (size_t)g * p.D + i];
        qv = p.q[(size_t)(tb + b) * p.q_stride + (size_t)g * p.D + i];
        if (p.silu_in) { kv = ms_silu(kv); qv = ms_silu(qv); }
      }
      ks[x] = kv;
      qs[x] = qv;
    }
    for (int x = tid; x < MS_BATCH * p.cols; x += blockDim.x) {
      const int b = x / p.cols, c = blockIdx.z * p.cols + x % p.cols;
      float vv = 0.0f;
      if (b < nb && c < p.V) {
        vv = p.v[(size_t)(tb + b) * p.v_stride + (size_t)h * p.V + c];
        if (p.silu_in) vv = ms_silu(vv);
      }
      vs[x] = vv;
    }
    if (MODE == MS_DELTA && tid < 2 * MS_BATCH) {
      const int b = tid >> 1, which = tid & 1;
      gs[tid] = b < nb ? p.gates[(size_t)(tb + b) * p.gates_stride + which * p.H + h] : 0.0f;
    }
    __syncthreads();
    for (int b = 0; b < nb; b++) {
      const float* kr = ks + b * DP + sub;
      const float* qr = qs + b * DP + sub;
      const float vv = vs[b * p.cols + min(tid / L, p.cols - 1)];
      float kk[MS_PER];
#pragma unroll
      for (int e = 0; e < MS_PER; e++) kk[e] = kr[e * L];
      float o = 0.0f;
      if (MODE == MS_DELTA) {
        float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          d0 = fmaf(S[e], kk[e], d0);
          d1 = fmaf(S[e + 1], kk[e + 1], d1);
          d2 = fmaf(S[e + 2], kk[e + 2], d2);
          d3 = fmaf(S[e + 3], kk[e + 3], d3);
        }
        float dk = (d0 + d1) + (d2 + d3);
#pragma unroll
        for (int m = 1; m < L; m <<= 1) dk += __shfl_xor_sync(0xffffffffu, dk, m);
        const float beta = gs[2 * b], gd = gs[2 * b + 1];
        const float u = beta * (vv - gd * dk);
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], u, gd * S[e]);
          S[e + 1] = fmaf(kk[e + 1], u, gd * S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], u, gd * S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], u, gd * S[e + 3]);
          o0 = fmaf(S[e], qr[e * L], o0);
          o1 = fmaf(S[e + 1], qr[(e + 1) * L], o1);
          o2 = fmaf(S[e + 2], qr[(e + 2) * L], o2);
          o3 = fmaf(S[e + 3], qr[(e + 3) * L], o3);
        }
        o = (o0 + o1) + (o2 + o3);
      } else {
        float o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
#pragma unroll
        for (int e = 0; e < MS_PER; e += 4) {
          S[e] = fmaf(kk[e], vv, hd * S[e]);
          S[e + 1] = fmaf(kk[e + 1], vv, hd * S[e + 1]);
          S[e + 2] = fmaf(kk[e + 2], vv, hd * S[e + 2]);
          S[e + 3] = fmaf(kk[e + 3], vv, hd * S[e + 3]);
          o0 = fmaf(S[e], qr[e * L], o0);
          o1 = fmaf(S[e + 1], qr[(e + 1) * L], o1);
          o2 = fmaf(S[e + 2], qr[(e + 2) * L], o2);
          o3 = fmaf(S[e + 3], qr[(e + 3) * L], o3);
        }
        o = (o0 + o1) + (o2 + o3);
      }
#pragma unroll
      for (int m = 1; m < L; m <<= 1) o += __shfl_xor_sync(0xffffffffu, o, m);
      if (on && sub == 0) p.out[(size_t)(tb + b) * p.out_stride + (size_t)h * p.V + col] = o;
    }
  }
#pragma unroll
  for (int e = 0; e < MS_PER; e++) {
    const int i = e * L + sub;
    if (on && i < p.D) sp[(size_t)i * p.V + col] = S[e];
  }
}

template <int MODE>
static int ms_launch(const MsArgs& p, int L, dim3 grid, int threads, size_t smem, cudaStream_t stream) {
  switch (L) {
    case 1: return sglc_launch(matrix_state_kernel<1, MODE>, grid, dim3(threads), smem, stream, 1, true, p);
    case 2: return sglc_launch(matrix_state_kernel<2, MODE>, grid, dim3(threads), smem, stream, 1, true, p);
    case 4: return sglc_launch(matrix_state_kernel<4, MODE>, grid, dim3(threads), smem, stream, 1, true, p);
    case 8: return sglc_launch(matrix_state_kernel<8, MODE>, grid, dim3(threads), smem, stream, 1, true, p);
  }
  return SGLC_ERR_UNSUPPORTED;
}

// mode 0: decay form (head_decay [H]); mode 1: gated delta rule (gates [T][2H]: beta, decay).
// q, k: float rows with G heads of D; v: H heads of V; out: [T][H*V] float; state [n_slots][H][D][V].
SGLC_API int sglc_matrix_state(int mode, const float* q, long long q_stride, const float* k, long long k_stride,
                               const float* v, long long v_stride, const float* gates, long long gates_stride,
                               const float* head_decay, float* out, long long out_stride, float* state,
                               int n_slots, const int* q_start, const int* state_slots, int R, int H, int G,
                               int D, int V, int silu_in, int* err, cudaStream_t stream) {
  if (R <= 0) return SGLC_OK;
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || V <= 0) return SGLC_ERR_ARGUMENT;
  if (D > MS_PER * 8 || H > 65535) return SGLC_ERR_UNSUPPORTED;
  int L = 1;
  while (MS_PER * L < D) L <<= 1;
  MsArgs p = {};
  p.q = q; p.q_stride = q_stride; p.k = k; p.k_stride = k_stride; p.v = v; p.v_stride = v_stride;
  p.gates = gates; p.gates_stride = gates_stride; p.head_decay = head_decay;
  p.out = out; p.out_stride = out_stride; p.state = state; p.q_start = q_start; p.state_slots = state_slots;
  p.R = R; p.H = H; p.G = G; p.D = D; p.V = V; p.n_slots = n_slots; p.silu_in = silu_in; p.err = err;
  // a warp's worth of columns a block (the fewer columns, the more blocks share a request's tokens)
  p.cols = V < 32 / L ? V : 32 / L;
  const int threads = ((p.cols * L + 31) / 32) * 32;
  const int zb = (V + p.cols - 1) / p.cols;
  if (zb > 65535) return SGLC_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)2 * MS_BATCH * MS_PER * L + (size_t)MS_BATCH * p.cols + 2 * MS_BATCH) * sizeof(float);
  const dim3 grid(R, H, zb);
  if (mode == MS_DECAY) {
    if (!head_decay) return SGLC_ERR_ARGUMENT;
    return ms_launch<MS_DECAY>(p, L, grid, threads, smem, stream);
  }
  if (mode == MS_DELTA) {
    if (!gates) return SGLC_ERR_ARGUMENT;
    return ms_launch<MS_DELTA>(p, L, grid, threads, smem, stream);
  }
  return SGLC_ERR_ARGUMENT;
}
