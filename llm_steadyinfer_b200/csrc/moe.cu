// Routed feed-forward ("mixture of experts"): every row chooses `top` of E small feed-forwards by a score and adds their
// results, weighted. Everything that depends on the choice happens on the device: no count travels to the host, so a
// step through these kernels can be recorded in a graph.
//   moe_route    scores z = W_r x (fp32 sums over the row in fp32), s = sigmoid(z) (or softmax over the experts), the `top`
//                largest (ties: the lower index), weights s * scale (optionally divided by their sum); rows of further
//                gate matrices behind the router's give sigmoid(w . x) for the same row (a gate on a shared expert).
//                With a choice bias the `top` largest of s + bias are chosen instead; the weights stay s.
//   moe_plan     the (row, choice) pairs ordered by expert, rows in step order within an expert: offsets per expert, the
//                row of every place, the place of every pair. Counting ranks within chunks of 1,024 pairs, so the order
//                never depends on timing.
//   moe_gemm     C[place] = act(A[row of place] W_e^T) for every place of expert e: a grouped product whose row tiles are
//                found from the offsets by every block itself (blocks beyond the last tile leave). bf16 on mma.sync
//                m16n8k16 with fp32 sums, tiles of 64 or 16 rows x 64 columns, three cp.async stages; fp32 on FFMA.
//                act "glu_limited": W_e holds gate and up rows in turn (row 2i the gate of entry i, row 2i + 1 its up), and
//                C[place, i] = g sigmoid(alpha g) (u + 1) with g = min(gate sum, limit), u = clamp(up sum, -limit, limit).
//                A row's sums run over k in the same order wherever the row lies in its tile. (Many rows in bf16
//                go to the tcgen05 grouped product of gemm_tc05.cu instead, behind `moe_gather`.)
//   moe_combine  out[t] = sum_c weight[t, c] * Y[place(t, c)] (+ gate[t] * shared[t]), the choices in their own order.
//                A choice whose id is not below `real` names an identity expert: its result is the row x[t] itself.
#include "common.cuh"
#include <math.h>
#include <mma.h>

typedef __nv_bfloat16 bf16;

// ---- router -------------------------------------------------------------------------------------------------------------
// x [T, d]; w [E + extra, d] (router rows, then `extra` gate rows) in the compute dtype; ids int32 [T, top]; wts fp32
// [T, top]; gates fp32 [T, extra]. mode 0: sigmoid scores; 1: softmax over the experts. One block a row.
template <typename T>
__global__ void __launch_bounds__(256) moe_route_kernel(const T* __restrict__ x, long long x_stride, const T* __restrict__ w,
    int E, int extra, int d, int top, float scale, int mode, int renorm, const float* __restrict__ choice_bias,
    int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ gates) {
  extern __shared__ float rsm[];                       // the row [d], scores [E + extra], used [E], choice keys [E]
  pdl_prologue();
  float* xr = rsm;
  float* sc = rsm + d;
  float* used = sc + E + extra;
  float* key = used + E;
  const long long t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int i = threadIdx.x; i < d; i += blockDim.x) xr[i] = to_f32<T>(x[t * x_stride + i]);
  for (int e = threadIdx.x; e < E; e += blockDim.x) used[e] = 0.f;
  __syncthreads();
  for (int e = warp; e < E + extra; e += nwarps) {
    const T* we = w + (size_t)e * d;
    float acc = 0.f;
    if (sizeof(T) == 2 && d % 8 == 0 && ((uintptr_t)w & 15) == 0) {      // rows of 16-byte pieces: eight entries a load
      for (int i = lane * 8; i < d; i += 256) {
        const uint4 raw = *reinterpret_cast<const uint4*>(we + i);
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          acc = fmaf(f.x, xr[i + 2 * j], acc);
          acc = fmaf(f.y, xr[i + 2 * j + 1], acc);
        }
      }
    } else {
      for (int i = lane; i < d; i += 32) acc = fmaf(to_f32<T>(we[i]), xr[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) sc[e] = acc;
  }
  __syncthreads();
  if (warp != 0) return;
  for (int e = lane; e < extra; e += 32) gates[t * extra + e] = 1.f / (1.f + expf(-sc[E + e]));
  float zmax = -INFINITY, zsum = 0.f;
  if (mode == 1) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, sc[e]);
    zmax = warp_max(zmax);
    for (int e = lane; e < E; e += 32) zsum += expf(sc[e] - zmax);
    zsum = warp_sum(zsum);
  }
  // what the choice goes by: the sums themselves (the scores rise with them), or score + bias where a bias is given
  for (int e = lane; e < E; e += 32) {
    float kv = sc[e];
    if (choice_bias) kv = (mode == 1 ? expf(sc[e] - zmax) / zsum : 1.f / (1.f + expf(-sc[e]))) + choice_bias[e];
    key[e] = kv;
  }
  __syncwarp();
  float total = 0.f, mine = 0.f;
  int my_id = 0;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int idx = -1;
    for (int e = lane; e < E; e += 32)
      if (used[e] == 0.f && (idx < 0 || key[e] > best)) { best = key[e]; idx = e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (oi >= 0 && (idx < 0 || ob > best || (ob == best && oi < idx))) { best = ob; idx = oi; }
    }
    if (idx < 0) idx = 0;                              // fewer experts than choices: never with a checked configuration
    const float z = sc[idx];
    const float s = mode == 1 ? expf(z - zmax) / zsum : 1.f / (1.f + expf(-z));
    total += s;
    if (lane == c % 32 && c < 32) { mine = s; my_id = idx; }
    if (lane == 0) used[idx] = 1.f;
    __syncwarp();
  }
  if (lane < top) {
    ids[t * top + lane] = my_id;
    wts[t * top + lane] = (renorm ? mine / total : mine) * scale;
  }
}

SI_EXPORT int si_moe_route(const void* x, int dtype, long long x_stride, const void* w, int E, int extra, int d, int top,
                           float scale, int mode, int renorm, const float* choice_bias, int* ids, float* wts, float* gates,
                           int rows, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E || top > 32 || extra < 0 || d <= 0 || mode < 0 || mode > 1) return -2;
  const size_t smem = (size_t)(d + 3 * E + extra) * sizeof(float);
  if (smem > 160 * 1024) return -2;
  const dim3 grid(rows), block(E + extra >= 8 ? 256 : 128);
#define ROUTE_LAUNCH(T)                                                                                                \
  {                                                                                                                  \
    static size_t configured = 0;                                                                                    \
    if (smem > 48 * 1024 && smem > configured) {                                                                     \
      if (cudaFuncSetAttribute(moe_route_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -2; \
      configured = smem;                                                                                             \
    }                                                                                                                \
    si_launch(moe_route_kernel<T>, grid, block, smem, stream, (const T*)x, x_stride, (const T*)w, E, extra, d, top, scale, \
              mode, renorm, choice_bias, ids, wts, gates);                                                           \
  }
  if (dtype == SI_BF16) ROUTE_LAUNCH(bf16) else ROUTE_LAUNCH(float)
#undef ROUTE_LAUNCH
  return si_last_error();
}

// ---- plan ---------------------------------------------------------------------------------------------------------------
#define PLAN_CHUNK 1024

// One chunk of pairs: every pair's rank among the pairs of the same expert before it in the chunk, and the chunk's count
// per expert.
__device__ void plan_rank_chunk(const int* __restrict__ ids, int P, int E, int chunk, int* __restrict__ rank,
                                int* __restrict__ counts, int* sm_ids) {
  const int base = chunk * PLAN_CHUNK;
  const int n = min(PLAN_CHUNK, P - base);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int e = ids[base + i];
    sm_ids[i] = (e < 0 || e >= E) ? 0 : e;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int e = sm_ids[i];
    int r = 0;
    for (int j = 0; j < i; ++j) r += sm_ids[j] == e;
    rank[base + i] = r;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int j = 0; j < n; ++j) c += sm_ids[j] == e;
    counts[(size_t)chunk * E + e] = c;
  }
}

// counts [chunks, E] become the first place of every (chunk, expert); offsets [E + 1] the first place of every expert.
__device__ void plan_offsets(int* __restrict__ counts, int chunks, int E, int* __restrict__ offsets, int* sm_tot) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int k = 0; k < chunks; ++k) c += counts[(size_t)k * E + e];
    sm_tot[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { const int c = sm_tot[e]; sm_tot[e] = acc; offsets[e] = acc; acc += c; }
    offsets[E] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int acc = sm_tot[e];
    for (int k = 0; k < chunks; ++k) { const int c = counts[(size_t)k * E + e]; counts[(size_t)k * E + e] = acc; acc += c; }
  }
}

__device__ void plan_place(const int* __restrict__ ids, const int* __restrict__ rank, const int* __restrict__ counts, int P,
                           int E, int top, int first, int last, int* __restrict__ row_of, int* __restrict__ place_of) {
  for (int i = first + threadIdx.x; i < last; i += blockDim.x) {
    int e = ids[i];
    e = (e < 0 || e >= E) ? 0 : e;
    const int place = counts[(size_t)(i / PLAN_CHUNK) * E + e] + rank[i];
    row_of[place] = i / top;
    place_of[i] = place;
  }
}

__global__ void __launch_bounds__(1024) moe_plan_one_kernel(const int* __restrict__ ids, int P, int E, int top,
    int* __restrict__ rank, int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ row_of,
    int* __restrict__ place_of) {
  extern __shared__ int psm[];                         // ids of the chunk [PLAN_CHUNK], totals [E]
  pdl_prologue();
  plan_rank_chunk(ids, P, E, 0, rank, counts, psm);
  __syncthreads();
  plan_offsets(counts, 1, E, offsets, psm + PLAN_CHUNK);
  __syncthreads();
  plan_place(ids, rank, counts, P, E, top, 0, P, row_of, place_of);
}
__global__ void __launch_bounds__(1024) moe_plan_rank_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ rank,
                                                             int* __restrict__ counts) {
  extern __shared__ int psm[];
  pdl_prologue();
  plan_rank_chunk(ids, P, E, blockIdx.x, rank, counts, psm);
}
__global__ void __launch_bounds__(1024) moe_plan_offsets_kernel(int* __restrict__ counts, int chunks, int E, int* __restrict__ offsets) {
  extern __shared__ int psm[];
  pdl_prologue();
  plan_offsets(counts, chunks, E, offsets, psm);
}
__global__ void __launch_bounds__(1024) moe_plan_place_kernel(const int* __restrict__ ids, const int* __restrict__ rank,
    const int* __restrict__ counts, int P, int E, int top, int* __restrict__ row_of, int* __restrict__ place_of) {
  pdl_prologue();
  const int first = blockIdx.x * PLAN_CHUNK;
  plan_place(ids, rank, counts, P, E, top, first, min(P, first + PLAN_CHUNK), row_of, place_of);
}

SI_EXPORT long long si_moe_plan_ints(int P, int E) {        // scratch of the plan: ranks, then counts per chunk
  const long long chunks = (P + PLAN_CHUNK - 1) / PLAN_CHUNK;
  return (long long)P + chunks * E;
}

SI_EXPORT int si_moe_plan(const int* ids, int P, int E, int top, int* scratch, int* offsets, int* row_of, int* place_of,
                          cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || E > 8192 || top <= 0 || P % top) return -2;
  const int chunks = (P + PLAN_CHUNK - 1) / PLAN_CHUNK;
  int* rank = scratch;
  int* counts = scratch + P;
  const int threads = P >= PLAN_CHUNK ? 1024 : ((P + 31) / 32) * 32;
  if (chunks == 1) {
    si_launch(moe_plan_one_kernel, dim3(1), dim3(threads), (size_t)(PLAN_CHUNK + E) * sizeof(int), stream, ids, P, E, top, rank,
              counts, offsets, row_of, place_of);
  } else {
    si_launch(moe_plan_rank_kernel, dim3(chunks), dim3(1024), (size_t)PLAN_CHUNK * sizeof(int), stream, ids, P, E, rank, counts);
    si_launch(moe_plan_offsets_kernel, dim3(1), dim3(E >= 512 ? 1024 : 256), (size_t)E * sizeof(int), stream, counts, chunks, E,
              offsets);
    si_launch(moe_plan_place_kernel, dim3(chunks), dim3(1024), 0, stream, ids, (const int*)rank, (const int*)counts, P, E, top,
              row_of, place_of);
  }
  return si_last_error();
}

// ---- grouped product ------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float moe_act(float v, int act) {
  if (act == 1) { const float r = fmaxf(v, 0.f); return r * r; }           // the square of relu
  if (act == 2) return v / (1.f + expf(-v));                               // silu
  if (act == 3) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));   // gelu_tanh
  return v;
}
#define MOE_ACT_GLU_LIMITED 4
// gate and up sums of one entry (neighbouring columns of the product): g sigmoid(alpha g) (u + 1) within the limit
__device__ __forceinline__ float moe_glu_limited(float gate, float up, float limit, float alpha) {
  const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + 1.f);
}

// The tile a block takes: expert, first place, places. Thread 0 walks the offsets; false: no tile is left for this block.
__device__ __forceinline__ bool moe_find_tile(const int* __restrict__ offsets, int E, int BM, int tile, int* sm3) {
  if (threadIdx.x == 0) {
    int acc = 0, found = -1, first = 0, rows = 0;
    for (int e = 0; e < E; ++e) {
      const int a = offsets[e], cnt = offsets[e + 1] - a;
      const int tiles = (cnt + BM - 1) / BM;
      if (tile < acc + tiles) { found = e; first = a + (tile - acc) * BM; rows = min(BM, a + cnt - first); break; }
      acc += tiles;
    }
    sm3[0] = found; sm3[1] = first; sm3[2] = rows;
  }
  __syncthreads();
  return sm3[0] >= 0;
}

#define MOE_BN 64
// A tile row in shared memory holds BK + 8 bf16 entries (fragment loads without bank conflicts). Tiles of 16 places stream
// an expert's weights for a handful of rows: 64 entries of k a stage and four stages keep enough bytes in flight; tiles of
// 64 places take 32 and three (static shared memory).

__device__ __forceinline__ void moe_cp16(void* dst, const void* src, int bytes) {       // bytes < 16: the rest is zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src), "r"(bytes));
}

// A [*, K] rows (row of place p: a_rows[p], or p itself when a_rows is absent); W [E, N, K]; C [places, N] (bf16 or fp32).
template <int BM, int BN, int MOE_BK, int MOE_STAGES>
__global__ void __launch_bounds__(128) moe_gemm_bf16_kernel(const bf16* __restrict__ A, long long a_stride,
    const int* __restrict__ a_rows, const bf16* __restrict__ W, void* __restrict__ C, long long c_stride, int c_f32,
    const int* __restrict__ offsets, int E, int N, int K, int act, int wide, float limit, float alpha) {
  constexpr int MOE_PITCH = MOE_BK + 8, KC = MOE_BK / 8;
  __shared__ __align__(16) bf16 As[MOE_STAGES][BM][MOE_PITCH];
  __shared__ __align__(16) bf16 Ws[MOE_STAGES][BN][MOE_PITCH];
  __shared__ int tile_info[3];
  __shared__ int src_row[BM];
  pdl_prologue();
  if (!moe_find_tile(offsets, E, BM, blockIdx.x, tile_info)) return;
  const int e = tile_info[0], first = tile_info[1], rows = tile_info[2];
  const int n0 = blockIdx.y * BN;
  for (int r = threadIdx.x; r < BM; r += blockDim.x) src_row[r] = r < rows ? (a_rows ? a_rows[first + r] : first + r) : -1;
  __syncthreads();
  const bf16* We = W + (size_t)e * N * K;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, tq = lane & 3;
  constexpr int NT = BM == 64 ? BN / 8 : BN / 32;    // n-tiles of 8 columns a warp: warps over the rows, or over the columns
  const int wr0 = BM == 64 ? warp * 16 : 0, wn0 = BM == 64 ? 0 : warp * (BN / 4);
  float acc[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  const int ktiles = (K + MOE_BK - 1) / MOE_BK;
  auto load = [&](int kt, int buf) {
    const int k0 = kt * MOE_BK;
    if (wide) {
      for (int c = threadIdx.x; c < (BM + BN) * KC; c += blockDim.x) {
        const int r = c / KC, kc = (c % KC) * 8;
        const int left = K - (k0 + kc);
        const int bytes = left >= 8 ? 16 : (left > 0 ? left * 2 : 0);
        if (r < BM) {
          const int sr = src_row[r];
          const bf16* src = sr >= 0 ? A + (size_t)sr * a_stride + k0 + kc : A;
          moe_cp16(&As[buf][r][kc], bytes > 0 ? src : A, sr >= 0 ? bytes : 0);
        } else {
          const int n = n0 + r - BM;
          const bf16* src = We + (size_t)(n < N ? n : 0) * K + k0 + kc;
          moe_cp16(&Ws[buf][r - BM][kc], bytes > 0 ? src : We, n < N ? bytes : 0);
        }
      }
    } else {                                           // rows that are not 16-byte aligned: entry by entry
      for (int c = threadIdx.x; c < (BM + BN) * MOE_BK; c += blockDim.x) {
        const int r = c / MOE_BK, kk = c % MOE_BK;
        const bool kin = k0 + kk < K;
        if (r < BM) {
          const int sr = src_row[r];
          As[buf][r][kk] = (sr >= 0 && kin) ? A[(size_t)sr * a_stride + k0 + kk] : __float2bfloat16_rn(0.f);
        } else {
          const int n = n0 + r - BM;
          Ws[buf][r - BM][kk] = (n < N && kin) ? We[(size_t)n * K + k0 + kk] : __float2bfloat16_rn(0.f);
        }
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  for (int s = 0; s < MOE_STAGES - 1; ++s) {
    if (s < ktiles) load(s, s);
    else asm volatile("cp.async.commit_group;\n" ::);
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(MOE_STAGES - 2) : "memory");
    __syncthreads();
    if (kt + MOE_STAGES - 1 < ktiles) load(kt + MOE_STAGES - 1, (kt + MOE_STAGES - 1) % MOE_STAGES);
    else asm volatile("cp.async.commit_group;\n" ::);
    const int buf = kt % MOE_STAGES;
#pragma unroll
    for (int kk = 0; kk < MOE_BK; kk += 16) {
      unsigned a0 = *reinterpret_cast<const unsigned*>(&As[buf][wr0 + g][kk + 2 * tq]);
      unsigned a1 = *reinterpret_cast<const unsigned*>(&As[buf][wr0 + g + 8][kk + 2 * tq]);
      unsigned a2 = *reinterpret_cast<const unsigned*>(&As[buf][wr0 + g][kk + 8 + 2 * tq]);
      unsigned a3 = *reinterpret_cast<const unsigned*>(&As[buf][wr0 + g + 8][kk + 8 + 2 * tq]);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int nn = wn0 + nt * 8 + g;
        unsigned b0 = *reinterpret_cast<const unsigned*>(&Ws[buf][nn][kk + 2 * tq]);
        unsigned b1 = *reinterpret_cast<const unsigned*>(&Ws[buf][nn][kk + 8 + 2 * tq]);
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                     : "+f"(acc[nt][0]), "+f"(acc[nt][1]), "+f"(acc[nt][2]), "+f"(acc[nt][3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
      }
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = wr0 + g + half * 8;
      if (r >= rows) continue;
      const size_t place = (size_t)(first + r);
      if (act == MOE_ACT_GLU_LIMITED) {                 // the thread's two columns are an entry's gate and up
        const int n = n0 + wn0 + nt * 8 + 2 * tq;
        if (n + 1 >= N) continue;
        const float v = moe_glu_limited(acc[nt][half * 2], acc[nt][half * 2 + 1], limit, alpha);
        if (c_f32) reinterpret_cast<float*>(C)[place * c_stride + (n >> 1)] = v;
        else reinterpret_cast<bf16*>(C)[place * c_stride + (n >> 1)] = __float2bfloat16_rn(v);
        continue;
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int n = n0 + wn0 + nt * 8 + 2 * tq + c;
        if (n >= N) continue;
        const float v = moe_act(acc[nt][half * 2 + c], act);
        if (c_f32) reinterpret_cast<float*>(C)[place * c_stride + n] = v;
        else reinterpret_cast<bf16*>(C)[place * c_stride + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

// True 32-bit: tiles of 32 places x 64 columns, 16 entries of k at a time, a thread 2 x 4 results.
__global__ void __launch_bounds__(256) moe_gemm_f32_kernel(const float* __restrict__ A, long long a_stride,
    const int* __restrict__ a_rows, const float* __restrict__ W, float* __restrict__ C, long long c_stride,
    const int* __restrict__ offsets, int E, int N, int K, int act, float limit, float alpha) {
  constexpr int BM = 32, BK = 16;
  __shared__ float As[BK][BM + 1];
  __shared__ float Ws[BK][MOE_BN + 1];
  __shared__ int tile_info[3];
  __shared__ int src_row[BM];
  pdl_prologue();
  if (!moe_find_tile(offsets, E, BM, blockIdx.x, tile_info)) return;
  const int e = tile_info[0], first = tile_info[1], rows = tile_info[2];
  const int n0 = blockIdx.y * MOE_BN;
  for (int r = threadIdx.x; r < BM; r += blockDim.x) src_row[r] = r < rows ? (a_rows ? a_rows[first + r] : first + r) : -1;
  __syncthreads();
  const float* We = W + (size_t)e * N * K;
  const int ty = threadIdx.x / 16, tx = threadIdx.x % 16;
  float acc[2][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int c = threadIdx.x; c < (BM + MOE_BN) * BK; c += blockDim.x) {
      const int r = c / BK, kk = c % BK;
      const bool kin = k0 + kk < K;
      if (r < BM) {
        const int sr = src_row[r];
        As[kk][r] = (sr >= 0 && kin) ? A[(size_t)sr * a_stride + k0 + kk] : 0.f;
      } else {
        const int n = n0 + r - BM;
        Ws[kk][r - BM] = (n < N && kin) ? We[(size_t)n * K + k0 + kk] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float a0 = As[kk][ty * 2], a1 = As[kk][ty * 2 + 1];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float b = Ws[kk][tx * 4 + c];
        acc[0][c] = fmaf(a0, b, acc[0][c]);
        acc[1][c] = fmaf(a1, b, acc[1][c]);
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = ty * 2 + rr;
    if (r >= rows) continue;
    if (act == MOE_ACT_GLU_LIMITED) {
#pragma unroll
      for (int c = 0; c < 4; c += 2) {
        const int n = n0 + tx * 4 + c;
        if (n + 1 < N) C[(size_t)(first + r) * c_stride + (n >> 1)] = moe_glu_limited(acc[rr][c], acc[rr][c + 1], limit, alpha);
      }
      continue;
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx * 4 + c;
      if (n < N) C[(size_t)(first + r) * c_stride + n] = moe_act(acc[rr][c], act);
    }
  }
}

SI_EXPORT int si_moe_gemm(const void* A, int dtype, long long a_stride, const int* a_rows, const void* W, void* C, int c_dtype,
                          long long c_stride, const int* offsets, int P, int E, int N, int K, int act, float limit, float alpha,
                          cudaStream_t stream) {
  if (P <= 0) return 0;
  if (E <= 0 || N <= 0 || K <= 0 || act < 0 || act > MOE_ACT_GLU_LIMITED) return -2;
  if (act == MOE_ACT_GLU_LIMITED && (N % 2 || !(limit > 0.f))) return -2;
  const int ny = (N + MOE_BN - 1) / MOE_BN;
  if (ny > 65535) return -2;
  if (dtype == SI_F32) {
    if (c_dtype != SI_F32) return -2;
    const dim3 grid((P + 31) / 32 + E, ny), block(256);
    si_launch(moe_gemm_f32_kernel, grid, block, 0, stream, (const float*)A, a_stride, a_rows, (const float*)W, (float*)C, c_stride,
              offsets, E, N, K, act, limit, alpha);
    return si_last_error();
  }
  const int wide = (K % 8 == 0 && a_stride % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0) ? 1 : 0;
  if (P < 32LL * E) {                                 // few rows an expert: tiles of 16 places
    // (32 columns a block, twice the blocks, measured no faster: 0.61 against 0.58 ms for the 16 launches of a decode step)
    const dim3 grid((P + 15) / 16 + E, ny), block(128);
    si_launch(moe_gemm_bf16_kernel<16, 64, 64, 4>, grid, block, 0, stream, (const bf16*)A, a_stride, a_rows, (const bf16*)W, C, c_stride,
              c_dtype == SI_F32 ? 1 : 0, offsets, E, N, K, act, wide, limit, alpha);
  } else {
    const dim3 grid((P + 63) / 64 + E, ny), block(128);
    si_launch(moe_gemm_bf16_kernel<64, 64, 32, 3>, grid, block, 0, stream, (const bf16*)A, a_stride, a_rows, (const bf16*)W, C, c_stride,
              c_dtype == SI_F32 ? 1 : 0, offsets, E, N, K, act, wide, limit, alpha);
  }
  return si_last_error();
}

// ---- rows in the order of their places ------------------------------------------------------------------------------------
// out[p, :] = a[rows[p], :] for every place p (what the TMA-fed grouped product reads as one matrix); 16 bytes a thread
// and step where rows are so aligned.
template <typename T>
__global__ void __launch_bounds__(256) moe_gather_kernel(const T* __restrict__ a, long long a_stride, const int* __restrict__ rows,
    T* __restrict__ out, long long out_stride, int num_rows, int K, int wide) {
  pdl_prologue();
  const long long p = blockIdx.x;
  int r = rows[p];
  if (r < 0 || r >= num_rows) r = 0;
  const T* src = a + (size_t)r * a_stride;
  T* dst = out + p * out_stride;
  if (wide) {
    constexpr int PER = 16 / sizeof(T);
    for (int i = threadIdx.x; i < K / PER; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
  }
}

SI_EXPORT int si_moe_gather(const void* a, int dtype, long long a_stride, const int* rows, void* out, long long out_stride,
                            int P, int num_rows, int K, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (K <= 0 || num_rows <= 0) return -2;
  const int es = dtype == SI_BF16 ? 2 : 4, per = 16 / es;
  const int wide = (K % per == 0 && a_stride % per == 0 && out_stride % per == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)out & 15) == 0) ? 1 : 0;
  const dim3 grid(P), block(K / per >= 256 ? 256 : 128);
  if (dtype == SI_BF16)
    si_launch(moe_gather_kernel<bf16>, grid, block, 0, stream, (const bf16*)a, a_stride, rows, (bf16*)out, out_stride, num_rows, K, wide);
  else
    si_launch(moe_gather_kernel<float>, grid, block, 0, stream, (const float*)a, a_stride, rows, (float*)out, out_stride, num_rows, K, wide);
  return si_last_error();
}

// ---- combine --------------------------------------------------------------------------------------------------------------
// out[t, :] = sum_c wts[t, c] * Y[place_of[t, c], :] + gate[t] * shared[t, :]   (gate absent: 1; shared absent: none)
// Y fp32 or the compute dtype; shared and out in the compute dtype. Sums in fp32, the choices in their own order.
template <typename TY, typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const TY* __restrict__ Y, long long y_stride, const int* __restrict__ place_of,
    const float* __restrict__ wts, int top, const T* __restrict__ shared, long long shared_stride, const float* __restrict__ gate,
    int gate_stride, T* __restrict__ out, long long out_stride, int d, const int* __restrict__ ids, int real,
    const T* __restrict__ x, long long x_stride) {
  pdl_prologue();
  const long long t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < d; i += blockDim.x * gridDim.y) {
    float acc = 0.f;
    for (int c = 0; c < top; ++c) {
      const bool same = ids && ids[t * top + c] >= real;           // an identity expert: the row itself
      const float y = same ? to_f32<T>(x[t * x_stride + i]) : to_f32<TY>(Y[(size_t)place_of[t * top + c] * y_stride + i]);
      acc = fmaf(wts[t * top + c], y, acc);
    }
    if (shared) acc = fmaf(gate ? gate[t * gate_stride] : 1.f, to_f32<T>(shared[t * shared_stride + i]), acc);
    out[t * out_stride + i] = from_f32<T>(acc);
  }
}

SI_EXPORT int si_moe_combine(const void* Y, int y_dtype, long long y_stride, const int* place_of, const float* wts, int top,
                             const void* shared, long long shared_stride, const float* gate, int gate_stride, void* out,
                             int dtype, long long out_stride, int rows, int d, const int* ids, int real, const void* x,
                             long long x_stride, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (top <= 0 || d <= 0 || (ids && !x)) return -2;
  const dim3 block(d >= 1024 ? 256 : 128);
  const dim3 grid(rows, si_row_shares(rows, d, block.x));
  if (dtype == SI_BF16 && y_dtype == SI_F32)
    si_launch(moe_combine_kernel<float, bf16>, grid, block, 0, stream, (const float*)Y, y_stride, place_of, wts, top,
              (const bf16*)shared, shared_stride, gate, gate_stride, (bf16*)out, out_stride, d, ids, real, (const bf16*)x, x_stride);
  else if (dtype == SI_BF16 && y_dtype == SI_BF16)
    si_launch(moe_combine_kernel<bf16, bf16>, grid, block, 0, stream, (const bf16*)Y, y_stride, place_of, wts, top,
              (const bf16*)shared, shared_stride, gate, gate_stride, (bf16*)out, out_stride, d, ids, real, (const bf16*)x, x_stride);
  else if (dtype == SI_F32 && y_dtype == SI_F32)
    si_launch(moe_combine_kernel<float, float>, grid, block, 0, stream, (const float*)Y, y_stride, place_of, wts, top,
              (const float*)shared, shared_stride, gate, gate_stride, (float*)out, out_stride, d, ids, real, (const float*)x, x_stride);
  else
    return -2;
  return si_last_error();
}
