// Attention of single decoded tokens over a cached latent: every head of a token reads the SAME
// rows (one shared key/value head, pages [n_pages][1][1][page_size][D]), so one block serves all
// heads of its token and brings each row from memory once, where a kernel with a block per
// (token, head) brings it once per head.
//
// A block owns a range of its token's keys (the keys are split over n_splits blocks) and a group
// of its heads (all of them when the launch has blocks enough without; else the heads are dealt to
// a few blocks, each of which then reads the range's rows), and walks the range in tiles of 64
// rows staged in shared memory as bfloat16:
//   scores   a thread a (head, key) pair: s = (q_h · c_j) * scale, 32-bit
//   softmax  online, a warp a head: m, l carried from tile to tile
//   values   a thread two adjacent columns of some heads' results: acc = acc * corr + sum_j p_j c_j
// With one range the result is normalised and written; with several, every range leaves
// (m, l, acc) in a workspace and a second small launch merges them in range order.
#include "common.cuh"

SGLC_DEFINE_ERROR_STRING()

namespace {
constexpr int THREADS = 256;
constexpr int WARPS = THREADS / 32;
constexpr int KT = 64;          // rows of a tile
constexpr int MAX_ACC = 8;      // pairs of columns a thread owns at most: H * D <= 2 * THREADS * MAX_ACC
constexpr int PAD = 8;          // bfloat16 of padding behind a staged row (keeps 16-byte loads of a quarter-warp apart)

struct LatentArgs {
  const __nv_bfloat16* q;
  int q_stride;
  const __nv_bfloat16* cache;
  const int* block_table;
  int bt_stride;
  const int* token_req;      // null: token t belongs to the step's t-th request
  const int* positions;
  const int* token_list;     // null: the launch serves tokens 0..T-1
  __nv_bfloat16* out;
  int o_stride;
  int H, D, page_size, window, n_splits, n_pages;
  int HG;                    // heads of a block (blockIdx.z deals the groups)
  float scale;
  float* ws;                 // [T][n_splits][H][D + 2] when n_splits > 1
  int* err;
};

__global__ void __launch_bounds__(THREADS)
latent_decode_kernel(LatentArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = a.D, RS = D + PAD;
  const int h0 = blockIdx.z * a.HG;                    // this block's heads: h0 .. h0 + H - 1
  const int H = min(a.HG, a.H - h0);
  __nv_bfloat16* rows = reinterpret_cast<__nv_bfloat16*>(smem_raw);            // [KT][RS]
  float* qs = reinterpret_cast<float*>(rows + (size_t)KT * RS);                // [H][D], scaled
  float* ps = qs + (size_t)a.HG * D;                                              // [H][KT]
  float* m_s = ps + (size_t)a.HG * KT;                                            // [H] running maximum
  float* l_s = m_s + a.HG;                                                        // [H] running sum
  float* c_s = l_s + a.HG;                                                        // [H] this tile's correction
  int* page_s = reinterpret_cast<int*>(c_s + a.HG);                               // [KT] page of each row of the tile
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot_t = blockIdx.x, sp = blockIdx.y;
  pdl_launch_dependents();
  // the step's own arrays were copied in before the step began: they may be read ahead of the wait
  const int t = a.token_list ? a.token_list[slot_t] : slot_t;
  const int r = a.token_req ? a.token_req[t] : t;
  const int pos = a.positions[t];
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  const int n = pos - lo + 1;
  const int chunk = (n + a.n_splits - 1) / a.n_splits;
  const int k0 = lo + sp * chunk;
  const int k1 = min(k0 + chunk, pos + 1);
  const int* bt = a.block_table + (size_t)r * a.bt_stride;
  for (int h = tid; h < H; h += THREADS) { m_s[h] = -INFINITY; l_s[h] = 0.0f; }
  const int n_pairs = H * D / 2;                       // (D is even)
  float2 acc[MAX_ACC];
#pragma unroll
  for (int i = 0; i < MAX_ACC; i++) acc[i] = make_float2(0.0f, 0.0f);
  pdl_wait();
  // queries (made by the kernel ahead), scaled once
  const __nv_bfloat16* qp = a.q + (size_t)t * a.q_stride + (size_t)h0 * D;
  for (int i = tid; i < H * D; i += THREADS) qs[i] = __bfloat162float(qp[i]) * a.scale;
  const int vec_per_row = D / 8;
  for (int key0 = k0; key0 < k1; key0 += KT) {
    const int nk = min(KT, k1 - key0);
    __syncthreads();                                   // the tile before has been used; qs, m, l are set
    if (tid < KT) {
      int page = -1;
      if (tid < nk) {
        page = bt[(key0 + tid) / a.page_size];
        if (!sglc_index_ok(page, a.n_pages, a.err)) page = -1;
      }
      page_s[tid] = page;
    }
    __syncthreads();
    for (int i = tid; i < KT * vec_per_row; i += THREADS) {
      const int j = i / vec_per_row, v = i % vec_per_row;
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      const int page = page_s[j];
      if (page >= 0)
        x = *(reinterpret_cast<const uint4*>(a.cache + ((size_t)page * a.page_size + (key0 + j) % a.page_size) * D) + v);
      *reinterpret_cast<uint4*>(rows + (size_t)j * RS + v * 8) = x;
    }
    __syncthreads();
    // scores: consecutive threads take consecutive keys of one head (the head's query is a broadcast)
    for (int i = tid; i < H * KT; i += THREADS) {
      const int h = i / KT, j = i % KT;
      const float* qh = qs + (size_t)h * D;
      const __nv_bfloat16* row = rows + (size_t)j * RS;
      float s0 = 0.0f, s1 = 0.0f;
      for (int d = 0; d < D; d += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(row + d);
        const float4 qa = *reinterpret_cast<const float4*>(qh + d), qb = *reinterpret_cast<const float4*>(qh + d + 4);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
        const float2 f0 = __bfloat1622float2(b2[0]), f1 = __bfloat1622float2(b2[1]);
        const float2 f2 = __bfloat1622float2(b2[2]), f3 = __bfloat1622float2(b2[3]);
        s0 = fmaf(qa.x, f0.x, s0); s1 = fmaf(qa.y, f0.y, s1);
        s0 = fmaf(qa.z, f1.x, s0); s1 = fmaf(qa.w, f1.y, s1);
        s0 = fmaf(qb.x, f2.x, s0); s1 = fmaf(qb.y, f2.y, s1);
        s0 = fmaf(qb.z, f3.x, s0); s1 = fmaf(qb.w, f3.y, s1);
      }
      ps[i] = j < nk ? s0 + s1 : -INFINITY;
    }
    __syncthreads();
    // online softmax: a warp a head
    for (int h = warp; h < H; h += WARPS) {
      float* p = ps + (size_t)h * KT;
      const float s_a = p[lane], s_b = p[lane + 32];
      const float m_old = m_s[h];
      const float m_new = fmaxf(m_old, warp_max(fmaxf(s_a, s_b)));
      const float e_a = expf(s_a - m_new), e_b = expf(s_b - m_new);      // (-inf: 0; a tile has at least one key)
      p[lane] = e_a;
      p[lane + 32] = e_b;
      const float sum = warp_sum(e_a + e_b);
      if (lane == 0) {
        const float corr = expf(m_old - m_new);                          // (first tile: exp(-inf) = 0)
        c_s[h] = corr;
        l_s[h] = l_s[h] * corr + sum;
        m_s[h] = m_new;
      }
    }
    __syncthreads();
    // values: a thread owns pairs of adjacent columns, pair index = i * THREADS + tid
#pragma unroll
    for (int i = 0; i < MAX_ACC; i++) {
      const int pair = i * THREADS + tid;
      if (pair < n_pairs) {
        const int h = (2 * pair) / D, d = (2 * pair) % D;
        const float corr = c_s[h];
        const float* p = ps + (size_t)h * KT;
        float ax = acc[i].x * corr, ay = acc[i].y * corr;
        for (int j = 0; j < nk; j++) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(rows + (size_t)j * RS + d));
          const float w = p[j];
          ax = fmaf(w, f.x, ax);
          ay = fmaf(w, f.y, ay);
        }
        acc[i] = make_float2(ax, ay);
      }
    }
  }
  __syncthreads();
  if (a.n_splits == 1) {
    __nv_bfloat16* op = a.out + (size_t)t * a.o_stride + (size_t)h0 * D;
#pragma unroll
    for (int i = 0; i < MAX_ACC; i++) {
      const int pair = i * THREADS + tid;
      if (pair < n_pairs) {
        const float inv = 1.0f / l_s[(2 * pair) / D];
        *reinterpret_cast<__nv_bfloat162*>(op + 2 * pair) = __floats2bfloat162_rn(acc[i].x * inv, acc[i].y * inv);
      }
    }
    return;
  }
  // several ranges: (acc, m, l) of this range, head by head
  float* w = a.ws + (((size_t)slot_t * a.n_splits + sp) * a.H + h0) * (D + 2);
#pragma unroll
  for (int i = 0; i < MAX_ACC; i++) {
    const int pair = i * THREADS + tid;
    if (pair < n_pairs) {
      const int h = (2 * pair) / D, d = (2 * pair) % D;
      *reinterpret_cast<float2*>(w + (size_t)h * (D + 2) + d) = acc[i];
    }
  }
  for (int h = tid; h < H; h += THREADS) {
    w[(size_t)h * (D + 2) + D] = m_s[h];
    w[(size_t)h * (D + 2) + D + 1] = l_s[h];
  }
}

// out[t][h][:] = sum_sp acc_sp * exp(m_sp - M) / sum_sp l_sp * exp(m_sp - M), ranges in order; a
// thread a column of a head, its loads asked for together
constexpr int MAX_SPLITS = 16;
__global__ void __launch_bounds__(THREADS)
latent_merge_kernel(LatentArgs a) {
  pdl_launch_dependents();
  const int slot_t = blockIdx.x;
  const int t = a.token_list ? a.token_list[slot_t] : slot_t;
  const int H = a.H, D = a.D;
  const int i = blockIdx.y * THREADS + threadIdx.x;
  pdl_wait();
  if (i >= H * D) return;
  const int h = i / D, d = i % D;
  const float* w = a.ws + ((size_t)slot_t * a.n_splits * H + h) * (D + 2);
  const size_t step = (size_t)H * (D + 2);
  float m[MAX_SPLITS], l[MAX_SPLITS], v[MAX_SPLITS];
#pragma unroll
  for (int sp = 0; sp < MAX_SPLITS; sp++) {
    const bool on = sp < a.n_splits;
    m[sp] = on ? w[sp * step + D] : -INFINITY;
    l[sp] = on ? w[sp * step + D + 1] : 0.0f;
    v[sp] = on ? w[sp * step + d] : 0.0f;
  }
  float M = -INFINITY;
#pragma unroll
  for (int sp = 0; sp < MAX_SPLITS; sp++) M = fmaxf(M, m[sp]);
  float L = 0.0f, o = 0.0f;
#pragma unroll
  for (int sp = 0; sp < MAX_SPLITS; sp++) {
    const float f = l[sp] > 0.0f ? expf(m[sp] - M) : 0.0f;      // (a range past the token's keys is empty)
    L = fmaf(l[sp], f, L);
    o = fmaf(v[sp], f, o);
  }
  a.out[(size_t)t * a.o_stride + i] = __float2bfloat16_rn(o / L);
}
}  // namespace

// Whether the kernel takes these sizes (else the caller uses the kernel with a block per head).
SGLC_API int sglc_attention_latent_decode_supports(int H, int D) {
  if (H <= 0 || D <= 0 || D % 8 != 0) return 0;
  if ((long long)H * D > 2LL * THREADS * MAX_ACC) return 0;
  const size_t smem = (size_t)KT * (D + PAD) * 2 + ((size_t)H * D + (size_t)H * KT + 3 * (size_t)H) * 4 + KT * 4;
  return smem <= 200 * 1024;
}

// Key ranges for T tokens with up to max_keys keys: enough blocks to fill the SMs, a range no
// shorter than one tile.
SGLC_API int sglc_attention_latent_decode_splits(int T, int max_keys) {
  int want = (148 + T - 1) / T;
  const int most = (max_keys + KT - 1) / KT;
  if (want > most) want = most;
  if (want > MAX_SPLITS) want = MAX_SPLITS;
  if (want < 1) want = 1;
  return want;
}

// q, out: bfloat16 [T][stride], heads side by side (H * D columns); cache: bfloat16 rows
// [n_pages][page_size][D]; positions[t]: the token's own position (its row is in the cache);
// T: tokens this launch serves (all, or the first T of token_list); ws: n_splits > 1 needs
// T * n_splits * H * (D + 2) floats.
SGLC_API int sglc_attention_latent_decode(const void* q, int q_stride, const void* cache, const int* block_table,
                                          int bt_stride, const int* token_req, const int* positions,
                                          const int* token_list, void* out, int o_stride, int T, int H, int D,
                                          int page_size, float scale, int window, int n_splits, float* ws,
                                          long long ws_floats, int n_pages, int* err, cudaStream_t stream) {
  if (T <= 0) return SGLC_OK;
  if (page_size <= 0 || n_splits < 1) return SGLC_ERR_ARGUMENT;
  if (!sglc_attention_latent_decode_supports(H, D) || n_splits > MAX_SPLITS) return SGLC_ERR_UNSUPPORTED;
  if (((uintptr_t)cache & 15) || ((uintptr_t)out & 3) || o_stride % 2 != 0) return SGLC_ERR_UNSUPPORTED;
  if (n_splits > 1 && (!ws || (long long)T * n_splits * H * (D + 2) > ws_floats)) return SGLC_ERR_ARGUMENT;
  LatentArgs a;
  a.q = (const __nv_bfloat16*)q; a.q_stride = q_stride;
  a.cache = (const __nv_bfloat16*)cache;
  a.block_table = block_table; a.bt_stride = bt_stride;
  a.token_req = token_req; a.positions = positions; a.token_list = token_list;
  a.out = (__nv_bfloat16*)out; a.o_stride = o_stride;
  a.H = H; a.D = D; a.page_size = page_size; a.window = window; a.n_splits = n_splits; a.n_pages = n_pages;
  a.scale = scale; a.ws = ws; a.err = err;
  // heads are dealt to several blocks while the launch has fewer than one and a half blocks an SM
  const long long base = (long long)T * n_splits;
  int groups = (int)((222 + base - 1) / base);
  if (groups > H) groups = H;
  a.HG = (H + groups - 1) / groups;
  groups = (H + a.HG - 1) / a.HG;
  const size_t smem = (size_t)KT * (D + PAD) * 2 + ((size_t)a.HG * D + (size_t)a.HG * KT + 3 * (size_t)a.HG) * 4 + KT * 4;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int rc = sglc_launch(latent_decode_kernel, dim3(T, n_splits, groups), dim3(THREADS), smem, stream, 1, true, a);
  if (rc != SGLC_OK || n_splits == 1) return rc;
  return sglc_launch(latent_merge_kernel, dim3(T, (H * D + THREADS - 1) / THREADS), dim3(THREADS), 0, stream, 1, true, a);
}
