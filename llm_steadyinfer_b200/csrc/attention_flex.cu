// bf16 attention over the paged cache on the tensor cores (mma.sync m16n8k16, fp32 accumulation, fp32 online
// softmax) in the general form of attention_general.cu: key size dk and value size dv of any multiple of 8,
// values of their own or the first dv entries of the keys (a latent that is key and value), a bias by distance
// added to the scaled score, an output gate (the result times sigmoid of a row of gate sums), a penalty slope[h] * (i - j) taken off it, a query temperature by position (row i's scale
// times 1 + coef * ln(floor((i + 1) / every) + 1)), a sink per head in the denominator, a soft limit on the scaled score
// (s <- cap * tanh(s / cap)), key heads that share a value head (v_share neighbouring key heads read one of the
// KV / v_share value heads), results in fp32 where the caller goes on computing with them. One kernel serves prompt
// portions and decode rows; for decode the key range of an item can be split over blocks, whose fp32 partial results a second small
// kernel merges.
//
// A work item is a run of consecutive query tokens of one sequence. A block handles one item, one KV head, one
// part of that KV head's query heads (Gb of them, so that tokens * Gb rows fit the 64-row tile; a latent shared
// by 128 heads is served in two parts), one slice of DVB value columns and one share of the keys. Row r of the
// tile is token r / Gb, head r % Gb; warp w owns rows 16w..16w+15 and walks all keys of the share. K tiles of
// BLOCK_N keys x dk come through cp.async into XOR-swizzled shared memory, two stages deep; the values are a
// second tile (own values: only the block's slice) or columns of the key tile itself.
// Sizes are run-time values: the loops over dk are not unrolled by the compiler, only the value slice (DVB, the
// accumulators) and the key tile (BLOCK_N) are template parameters.
#include "attention_common.cuh"

struct FlexParams {
  const bf16* q; long long q_stride;
  const bf16* k_cache; const bf16* v_cache;      // v_cache nullptr: values are keys[..., :dv]
  const int* block_table; int table_width;
  const AttnItem* items; int num_items;
  bf16* out; long long out_stride;
  float* out_f32;           // not null: results go here as fp32 (same strides), not to `out`
  float cap_log2, scale_over_cap;   // soft limit: cap * log2(e) and 2 * log2(e) * scale / cap (cap_log2 0: none)
  int v_share;              // key heads that read one value head
  float* part_o;            // [item][gy][split][64 rows][dv]   (nsplit > 1)
  float* part_ml;           // [item][gy][split][64 rows][2]
  const float* dist_bias; int nd;                // fp32 [nd, H] or nullptr
  const float* sink;                             // fp32 [H] or nullptr
  const float* slopes;                           // fp32 [H] or nullptr: slope[h] * distance leaves the scaled score
  float qt_coef; int qt_every;                   // query temperature (every 0: none)
  const bf16* gate; long long gate_stride;       // not null: the result (row, head, d) times sigmoid(gate[row, head * dv + d])
  int num_pages, page_size, num_seqs, H, KV, G, Gb, hparts, dk, dv, dk_pitch;
  int bias_in_smem;         // the distances a key tile can meet are staged in shared memory, tile by tile
  int warps_are_slices;     // items of at most 16 rows whose values are key columns: every warp takes rows 0..15 and a
                            // value slice of its own, so that a block serves four slices from one key tile
  float scale_log2;         // scale * log2(e)
  int window, nsplit;
  int* status;
};

#define FLEX_M 64
#define LOG2E 1.4426950408889634f

__device__ __forceinline__ bf16* ftile(bf16* base, int pitch_chunks, int row, int chunk) {
  return base + ((size_t)row * pitch_chunks + (chunk ^ (row & 7))) * 8;
}

// KSPLIT 4: items of at most 16 rows; every warp takes rows 0..15 and a quarter of each tile's keys, and the four
// partial results are merged through shared memory at the end.
template <int BLOCK_N, int DVB, int KSPLIT>
__global__ void __launch_bounds__(128)
attn_flex_kernel(const FlexParams p) {
  constexpr int THREADS = 128;
  constexpr int NT = BLOCK_N / 8 / KSPLIT;          // score n-tiles of a warp
  constexpr int KEYS_W = BLOCK_N / KSPLIT;          // keys of a tile that a warp takes
  constexpr int DT = DVB / 8;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int kch = p.dk_pitch / 8;                       // 16-byte chunks of a key row in shared memory
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
  bf16* Ks = Qs + (size_t)FLEX_M * p.dk_pitch;          // [2][BLOCK_N][dk_pitch]
  bf16* Vs = Ks + (size_t)2 * BLOCK_N * p.dk_pitch;     // [2][BLOCK_N][DVB]  (own values only)
  const bool own_v = p.v_cache != nullptr;
  // [2][BLOCK_N + 64 / Gb][Gb] biases of the distances that the rows of this block have to the keys of a tile
  float* Bs = reinterpret_cast<float*>(Vs + (own_v ? (size_t)2 * BLOCK_N * DVB : 0));
  const int bwin = BLOCK_N + FLEX_M / p.Gb;

  const int item_idx = blockIdx.x / p.nsplit, split = blockIdx.x % p.nsplit;
  const AttnItem item = p.items[item_idx];
  const int g = blockIdx.y / p.hparts, hpart = blockIdx.y % p.hparts;
  const int warp = threadIdx.x >> 5;
  const int wrow = (p.warps_are_slices || KSPLIT > 1) ? 0 : warp * 16;        // first tile row of this warp
  const int krow0 = KSPLIT > 1 ? warp * KEYS_W : 0;                           // first key row of a tile for this warp
  const int v0 = (p.warps_are_slices ? blockIdx.z * 4 + (threadIdx.x >> 5) : blockIdx.z) * DVB;   // first value column
  const int lane = threadIdx.x & 31;
  if (item.ntok <= 0) return;
  if (item.seq < 0 || item.seq >= p.num_seqs) {
    if (threadIdx.x == 0) set_status(p.status, SI_BAD_SEQ);
    return;
  }
  const int* table = p.block_table + (size_t)item.seq * p.table_width;
  const int kv_end_all = item.pos0 + item.ntok;
  const int kv_lo = window_first_key(item.pos0, p.window);
  const int kv_begin_all = kv_lo / BLOCK_N * BLOCK_N;
  const int tiles_all = (kv_end_all - kv_begin_all + BLOCK_N - 1) / BLOCK_N;
  const int tiles_per = (tiles_all + p.nsplit - 1) / p.nsplit;
  const int t_begin = split * tiles_per;
  const int t_end = min(tiles_all, t_begin + tiles_per);
  const int ntiles = max(0, t_end - t_begin);
  const int kv_begin = kv_begin_all + t_begin * BLOCK_N;
  const int kv_end = min(kv_end_all, kv_begin_all + t_end * BLOCK_N);
  const int head0 = g * p.G + hpart * p.Gb;
  const int dk_chunks = p.dk / 8;
  const int kt_steps = (p.dk + 15) / 16;

  // A thread fetches chunks of one key row per tile (THREADS / BLOCK_N threads share a row), so that the row's
  // page is looked up once per thread and tile; the copies that follow do not wait for one another.
  constexpr int TPR = THREADS / BLOCK_N;
  auto load_kv = [&](int j0, int stage) {
    bf16* Kt = Ks + (size_t)stage * BLOCK_N * p.dk_pitch;
    const int row = threadIdx.x / TPR, c_first = threadIdx.x % TPR;
    const int j = j0 + row;
    bool in_range = j >= kv_lo && j < kv_end;
    size_t tok = 0;
    if (in_range) {
      const int slot = j / p.page_size;
      const int page = slot < p.table_width ? table[slot] : -1;
      if (page < 0 || page >= p.num_pages) {
        set_status(p.status, SI_BAD_PAGE);
        in_range = false;
      } else {
        tok = ((size_t)page * p.KV + g) * p.page_size + (j - slot * p.page_size);
      }
    }
    const bf16* krow = p.k_cache + tok * p.dk;
    for (int c = c_first; c < kch; c += TPR) {
      const bool valid = in_range && c < dk_chunks;
      cp_async16(ftile(Kt, kch, row, c), valid ? krow + c * 8 : p.k_cache, valid);
    }
    if (own_v) {
      bf16* Vt = Vs + (size_t)stage * BLOCK_N * DVB;
      if (in_range && p.v_share > 1) {           // the value head that this key head shares with its neighbours
        const int slot = j / p.page_size;
        tok = ((size_t)table[slot] * (p.KV / p.v_share) + g / p.v_share) * p.page_size + (j - slot * p.page_size);
      }
      const bf16* vrow = p.v_cache + tok * p.dv + v0;
      for (int c = c_first; c < DT; c += TPR) {
        const bool valid = in_range && v0 + c * 8 < p.dv;
        cp_async16(ftile(Vt, DT, row, c), valid ? vrow + c * 8 : p.v_cache, valid);
      }
    }
    if (p.bias_in_smem) {                     // entry (d - dlo, head) with dlo the least distance of the tile
      float* Bt = Bs + (size_t)stage * bwin * p.Gb;
      const int dlo = item.pos0 - (j0 + BLOCK_N - 1);
      const int total = bwin * p.Gb;
      for (int id0 = threadIdx.x; id0 < total; id0 += 4 * THREADS) {        // four loads in flight, then four stores
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int id = id0 + u * THREADS;
          const int d = dlo + id / p.Gb;
          v[u] = (id < total && d >= 0) ? p.dist_bias[(size_t)min(d, p.nd - 1) * p.H + head0 + id % p.Gb] * LOG2E : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (id0 + u * THREADS < total) Bt[id0 + u * THREADS] = v[u];
      }
    }
  };

  if (ntiles > 0) {
    for (int id = threadIdx.x; id < FLEX_M * kch; id += THREADS) {
      const int row = id / kch, c = id % kch;
      const int tok = row / p.Gb, hh = row - tok * p.Gb;
      const bool valid = tok < item.ntok && c < dk_chunks;
      const bf16* src = p.q;
      if (valid) src = p.q + (size_t)(item.row0 + tok) * p.q_stride + (size_t)(head0 + hh) * p.dk + c * 8;
      cp_async16(ftile(Qs, kch, row, c), src, valid);
    }
    load_kv(kv_begin, 0);
  }
  cp_async_commit();

  const int r_lo = wrow + (lane >> 2), r_hi = r_lo + 8;
  const int tok_lo = r_lo / p.Gb, tok_hi = r_hi / p.Gb;
  const int pos_lo = tok_lo < item.ntok ? item.pos0 + tok_lo : -1;     // -1: row unused
  const int pos_hi = tok_hi < item.ntok ? item.pos0 + tok_hi : -1;
  const int hh_lo = r_lo % p.Gb, hh_hi = r_hi % p.Gb;
  const int head_lo = head0 + hh_lo, head_hi = head0 + hh_hi;
  // what a row's raw score is multiplied by beside the scale (its query temperature), and its head's slope (base 2)
  const float tf_lo = (p.qt_every > 0 && pos_lo >= 0) ? 1.f + p.qt_coef * logf((float)((pos_lo + 1) / p.qt_every + 1)) : 1.f;
  const float tf_hi = (p.qt_every > 0 && pos_hi >= 0) ? 1.f + p.qt_coef * logf((float)((pos_hi + 1) / p.qt_every + 1)) : 1.f;
  const float sl_lo = p.slopes ? p.slopes[head_lo] * LOG2E : 0.f, sl_hi = p.slopes ? p.slopes[head_hi] * LOG2E : 0.f;
  const int warp_last_tok = min(item.ntok - 1, (wrow + 15) / p.Gb);
  const int warp_first_tok = wrow / p.Gb;
  const bool warp_active = warp_first_tok < item.ntok && v0 < p.dv;
  const int warp_max_pos = item.pos0 + warp_last_tok;
  const int warp_min_pos = item.pos0 + warp_first_tok;

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;

  for (int t = 0; t < ntiles; ++t) {
    const int j0 = kv_begin + t * BLOCK_N;
    bf16* Kt = Ks + (size_t)(t & 1) * BLOCK_N * p.dk_pitch;
    if (t + 1 < ntiles) {
      load_kv(j0 + BLOCK_N, (t + 1) & 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    bool skip = !warp_active || j0 + krow0 > warp_max_pos;
    if (p.window > 0 && j0 + krow0 + KEYS_W - 1 <= warp_min_pos - p.window) skip = true;
    if (!skip) {
      float s[NT][4];
#pragma unroll
      for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
      for (int kk = 0; kk < kt_steps; ++kk) {
        unsigned a0, a1, a2, a3;
        ldsm_x4(a0, a1, a2, a3, ftile(Qs, kch, wrow + (lane & 7) + 8 * ((lane >> 3) & 1), kk * 2 + (lane >> 4)));
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          unsigned b0, b1, b2, b3;
          ldsm_x4(b0, b1, b2, b3, ftile(Kt, kch, krow0 + nt * 8 + (lane & 7) + 8 * (lane >> 4), kk * 2 + ((lane >> 3) & 1)));
          mma_bf16(s[nt], a0, a1, a2, a3, b0, b1);
          mma_bf16(s[nt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      float mx_lo = m_lo, mx_hi = m_hi;
      const float* Bt = Bs + (size_t)(t & 1) * bwin * p.Gb;
      const int dlo = item.pos0 - (j0 + BLOCK_N - 1);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + krow0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int pos = (e < 2) ? pos_lo : pos_hi;
          const bool vis = j >= kv_lo && j <= pos && (p.window <= 0 || j > pos - p.window);
          float v = -INFINITY;
          if (vis) {
            // tanh(y) = 1 - 2 / (exp(2 y) + 1): absolute error of some 1e-7, which is what counts for a score
            const float raw = s[nt][e] * ((e < 2) ? tf_lo : tf_hi);
            v = p.cap_log2 > 0.f ? p.cap_log2 * (1.f - __fdividef(2.f, exp2f(raw * p.scale_over_cap) + 1.f)) : raw * p.scale_log2;
            if (p.bias_in_smem) v += Bt[(pos - j - dlo) * p.Gb + ((e < 2) ? hh_lo : hh_hi)];
            else if (p.dist_bias) v += p.dist_bias[(size_t)min(pos - j, p.nd - 1) * p.H + ((e < 2) ? head_lo : head_hi)] * LOG2E;
            v -= ((e < 2) ? sl_lo : sl_hi) * (float)(pos - j);
          }
          s[nt][e] = v;
          if (e < 2) mx_lo = fmaxf(mx_lo, v); else mx_hi = fmaxf(mx_hi, v);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float base_lo = mx_lo == -INFINITY ? 0.f : mx_lo;
      const float base_hi = mx_hi == -INFINITY ? 0.f : mx_hi;
      const float corr_lo = exp2f(m_lo - base_lo), corr_hi = exp2f(m_hi - base_hi);
      m_lo = mx_lo; m_hi = mx_hi;
      float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - base_lo); s[nt][1] = exp2f(s[nt][1] - base_lo);
        s[nt][2] = exp2f(s[nt][2] - base_hi); s[nt][3] = exp2f(s[nt][3] - base_hi);
        sum_lo += s[nt][0] + s[nt][1];
        sum_hi += s[nt][2] + s[nt][3];
      }
      l_lo = l_lo * corr_lo + sum_lo;
      l_hi = l_hi * corr_hi + sum_hi;
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] *= corr_lo; o[i][1] *= corr_lo; o[i][2] *= corr_hi; o[i][3] *= corr_hi;
      }
      // O += P V: own values from their tile, else columns v0.. of the key tile
      bf16* Vt = own_v ? Vs + (size_t)(t & 1) * BLOCK_N * DVB : Kt;
      const int vch = own_v ? DT : kch;
      const int vc0 = own_v ? 0 : v0 / 8;
#pragma unroll
      for (int kk = 0; kk < KEYS_W / 16; ++kk) {
        const unsigned a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        const unsigned a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        const unsigned a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        const unsigned a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dt = 0; dt < DT; dt += 2) {
          if (v0 + dt * 8 >= p.dv) break;                 // columns beyond the values: nothing there to read
          unsigned b0, b1, b2, b3;
          ldsm_x4_t(b0, b1, b2, b3, ftile(Vt, vch, krow0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), vc0 + dt + (lane >> 4)));
          mma_bf16(o[dt], a0, a1, a2, a3, b0, b1);
          mma_bf16(o[dt + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();       // everyone is done with this stage before it is refilled
  }
  if (KSPLIT > 1) {
    // The warps hold partial results for the same rows and columns, lane by lane: warps 1.. hand theirs to warp 0
    // through shared memory (the tiles are done with), which weighs them by their maxima and goes on alone.
    constexpr int W = DT * 4 + 4;
    float* X = reinterpret_cast<float*>(smem_raw);
    if (warp > 0) {
      float* mine = X + (size_t)(warp - 1) * W * 32 + lane;
#pragma unroll
      for (int i = 0; i < DT; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) mine[(i * 4 + e) * 32] = o[i][e];
      mine[(DT * 4 + 0) * 32] = m_lo; mine[(DT * 4 + 1) * 32] = m_hi;
      mine[(DT * 4 + 2) * 32] = l_lo; mine[(DT * 4 + 3) * 32] = l_hi;
    }
    __syncthreads();
    if (warp > 0) return;
    float M_lo = m_lo, M_hi = m_hi;
#pragma unroll
    for (int w = 0; w < KSPLIT - 1; ++w) {
      M_lo = fmaxf(M_lo, X[((size_t)w * W + DT * 4 + 0) * 32 + lane]);
      M_hi = fmaxf(M_hi, X[((size_t)w * W + DT * 4 + 1) * 32 + lane]);
    }
    const float b_lo = M_lo == -INFINITY ? 0.f : M_lo, b_hi = M_hi == -INFINITY ? 0.f : M_hi;
    const float f_lo = exp2f(m_lo - b_lo), f_hi = exp2f(m_hi - b_hi);
    l_lo *= f_lo; l_hi *= f_hi;
#pragma unroll
    for (int i = 0; i < DT; ++i) { o[i][0] *= f_lo; o[i][1] *= f_lo; o[i][2] *= f_hi; o[i][3] *= f_hi; }
#pragma unroll
    for (int w = 0; w < KSPLIT - 1; ++w) {
      const float* theirs = X + (size_t)w * W * 32 + lane;
      const float g_lo = exp2f(theirs[(DT * 4 + 0) * 32] - b_lo), g_hi = exp2f(theirs[(DT * 4 + 1) * 32] - b_hi);
      l_lo = fmaf(theirs[(DT * 4 + 2) * 32], g_lo, l_lo);
      l_hi = fmaf(theirs[(DT * 4 + 3) * 32], g_hi, l_hi);
#pragma unroll
      for (int i = 0; i < DT; ++i) {
        o[i][0] = fmaf(theirs[(i * 4 + 0) * 32], g_lo, o[i][0]); o[i][1] = fmaf(theirs[(i * 4 + 1) * 32], g_lo, o[i][1]);
        o[i][2] = fmaf(theirs[(i * 4 + 2) * 32], g_hi, o[i][2]); o[i][3] = fmaf(theirs[(i * 4 + 3) * 32], g_hi, o[i][3]);
      }
    }
    m_lo = M_lo; m_hi = M_hi;
  }
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1); l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1); l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);

  if (p.nsplit > 1) {                       // partial results: unnormalised sums, maximum (base 2) and denominator
    const size_t slab = ((size_t)item_idx * gridDim.y + blockIdx.y) * p.nsplit + split;
    float* po = p.part_o + slab * FLEX_M * p.dv;
    float* pml = p.part_ml + slab * FLEX_M * 2;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? r_hi : r_lo;
      if (r / p.Gb >= item.ntok) continue;
      if ((lane & 3) == 0 && v0 == 0) {
        pml[r * 2] = half ? m_hi : m_lo;
        pml[r * 2 + 1] = half ? l_hi : l_lo;
      }
#pragma unroll
      for (int dt = 0; dt < DT; ++dt) {
        const int d = v0 + dt * 8 + (lane & 3) * 2;
        if (d < p.dv) *reinterpret_cast<float2*>(po + (size_t)r * p.dv + d) = make_float2(o[dt][half * 2], o[dt][half * 2 + 1]);
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = half ? r_hi : r_lo;
    const int tok = r / p.Gb, hh = r - tok * p.Gb;
    if (tok >= item.ntok) continue;
    float l = half ? l_hi : l_lo, f = 1.f;
    if (p.sink) {                           // exp(sink) joins the denominator once
      const float m = half ? m_hi : m_lo, s2 = p.sink[head0 + hh] * LOG2E;
      const float M = fmaxf(m, s2);
      f = exp2f(m - M);
      l = l * f + exp2f(s2 - M);
    }
    const float inv = l > 0.f ? f / l : 0.f;
    const size_t at = (size_t)(item.row0 + tok) * p.out_stride + (size_t)(head0 + hh) * p.dv;
    const bf16* grow = p.gate ? p.gate + (size_t)(item.row0 + tok) * p.gate_stride + (size_t)(head0 + hh) * p.dv : nullptr;
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      const int d = v0 + dt * 8 + (lane & 3) * 2;
      if (d >= p.dv) continue;
      float r0 = o[dt][half * 2] * inv, r1 = o[dt][half * 2 + 1] * inv;
      if (grow) {
        const float2 gz = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(grow + d));
        r0 /= 1.f + __expf(-gz.x); r1 /= 1.f + __expf(-gz.y);
      }
      if (p.out_f32) *reinterpret_cast<float2*>(p.out_f32 + at + d) = make_float2(r0, r1);
      else *reinterpret_cast<__nv_bfloat162*>(p.out + at + d) = __floats2bfloat162_rn(r0, r1);
    }
  }
}

// Merge of the shares of split items: one block per (item, gy, row); the first threads weigh the shares, then a
// thread per value column adds them up.
__global__ void attn_flex_merge_kernel(const FlexParams p) {
  __shared__ float w[64];
  __shared__ float s_inv;
  pdl_prologue();
  const AttnItem item = p.items[blockIdx.x];
  if (item.ntok <= 0 || item.seq < 0 || item.seq >= p.num_seqs) return;
  const int r = blockIdx.z;
  if (r >= item.ntok * p.Gb) return;
  const int g = blockIdx.y / p.hparts, hpart = blockIdx.y % p.hparts;
  const int tok = r / p.Gb, head = g * p.G + hpart * p.Gb + r % p.Gb;
  const size_t slab0 = ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * p.nsplit;
  if (threadIdx.x < 32) {                                 // nsplit <= 64: two shares a lane
    const int s0 = threadIdx.x, s1 = threadIdx.x + 32;
    const float m0 = s0 < p.nsplit ? p.part_ml[((slab0 + s0) * FLEX_M + r) * 2] : -INFINITY;
    const float m1 = s1 < p.nsplit ? p.part_ml[((slab0 + s1) * FLEX_M + r) * 2] : -INFINITY;
    const float sk = p.sink ? p.sink[head] * LOG2E : -INFINITY;
    const float M = fmaxf(warp_max(fmaxf(m0, m1)), sk);
    const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - M), w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - M);
    float L = (s0 < p.nsplit ? p.part_ml[((slab0 + s0) * FLEX_M + r) * 2 + 1] * w0 : 0.f)
            + (s1 < p.nsplit ? p.part_ml[((slab0 + s1) * FLEX_M + r) * 2 + 1] * w1 : 0.f);
    L = warp_sum(L) + (p.sink ? exp2f(sk - M) : 0.f);
    w[s0] = w0; w[s1] = w1;
    if (threadIdx.x == 0) s_inv = L > 0.f ? 1.f / L : 0.f;
  }
  __syncthreads();
  const size_t at = (size_t)(item.row0 + tok) * p.out_stride + (size_t)head * p.dv;
  for (int d = threadIdx.x; d < p.dv; d += blockDim.x) {
    float acc = 0.f;
    for (int s0 = 0; s0 < p.nsplit; s0 += 8) {            // eight loads in flight; shares without keys hold nothing
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = (s0 + u < p.nsplit && w[s0 + u] > 0.f) ? p.part_o[((slab0 + s0 + u) * FLEX_M + r) * p.dv + d] : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = fmaf(v[u], s0 + u < p.nsplit ? w[s0 + u] : 0.f, acc);
    }
    float res = acc * s_inv;
    if (p.gate) res /= 1.f + __expf(-__bfloat162float(p.gate[(size_t)(item.row0 + tok) * p.gate_stride + (size_t)head * p.dv + d]));
    if (p.out_f32) p.out_f32[at + d] = res;
    else p.out[at + d] = __float2bfloat16_rn(res);
  }
}

// ---- host side ------------------------------------------------------------------------------------------
static int flex_heads_per_block(int G) {          // the largest divisor of G that fits the 64-row tile
  for (int gb = G < FLEX_M ? G : FLEX_M; gb >= 1; --gb)
    if (G % gb == 0) return gb;
  return 1;
}

SI_EXPORT int si_attn_flex_ok(int H, int KV, int dk, int dv, int own_v) {
  if (H <= 0 || KV <= 0 || H % KV || dk <= 0 || dv <= 0 || dk % 8 || dv % 8 || dk > 640) return 0;
  if (!own_v && dv > dk) return 0;
  return 1;
}
// Most tokens of one item.
SI_EXPORT int si_attn_flex_tokens(int H, int KV) { return FLEX_M / flex_heads_per_block(H / KV); }
SI_EXPORT long long si_attn_flex_scratch_floats(int num_items, int H, int KV, int dv, int nsplit) {
  const int G = H / KV, gy = KV * (G / flex_heads_per_block(G));
  return (long long)num_items * gy * nsplit * FLEX_M * (dv + 2);
}

template <int BLOCK_N, int DVB, int KSPLIT>
static int flex_launch(const FlexParams& p, int dslices, size_t smem, cudaStream_t stream) {
  static size_t configured = 0;
  if (KSPLIT > 1 && smem < (size_t)(KSPLIT - 1) * 32 * (DVB / 2 + 4) * sizeof(float))
    smem = (size_t)(KSPLIT - 1) * 32 * (DVB / 2 + 4) * sizeof(float);          // room for the warps' merge
  if (smem > 48 * 1024 && smem > configured) {
    if (cudaFuncSetAttribute(attn_flex_kernel<BLOCK_N, DVB, KSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -2;
    configured = smem;
  }
  attn_flex_kernel<BLOCK_N, DVB, KSPLIT><<<dim3(p.num_items * p.nsplit, p.KV * p.hparts, dslices), 128, smem, stream>>>(p);
  return 0;
}

SI_EXPORT int si_attn_flex(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                           const int* block_table, int table_width, const int* items, int num_items, void* out,
                           long long out_stride, int num_pages, int page_size, int num_seqs, int H, int KV, int dk,
                           int dv, float scale, int window, const float* dist_bias, int nd, const float* sink,
                           int nsplit, float* scratch, int max_rows, float softcap, int v_share, int out_is_f32,
                           const float* slopes, float qt_coef, int qt_every, const void* gate, long long gate_stride,
                           int* status, cudaStream_t stream) {
  if (num_items <= 0) return 0;
  if (!si_attn_flex_ok(H, KV, dk, dv, v_cache != nullptr) || nsplit < 1 || nsplit > 64 || (nsplit > 1 && !scratch)) return -2;
  if (v_share < 1 || KV % v_share || (v_share > 1 && !v_cache) || softcap < 0.f || qt_every < 0) return -2;
  FlexParams p;
  p.slopes = slopes; p.qt_coef = qt_coef; p.qt_every = qt_every;
  p.gate = (const bf16*)gate; p.gate_stride = gate_stride;
  if (gate && (gate_stride % 2 || ((uintptr_t)gate & 3))) return -2;      // the gate is read two entries at a time
  p.q = (const bf16*)q; p.q_stride = q_stride;
  p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache;
  p.block_table = block_table; p.table_width = table_width;
  p.items = (const AttnItem*)items; p.num_items = num_items;
  p.out = out_is_f32 ? nullptr : (bf16*)out; p.out_stride = out_stride;
  p.out_f32 = out_is_f32 ? (float*)out : nullptr;
  p.cap_log2 = softcap > 0.f ? softcap * LOG2E : 0.f; p.scale_over_cap = softcap > 0.f ? 2.f * LOG2E * scale / softcap : 0.f;
  p.v_share = v_share;
  p.dist_bias = dist_bias; p.nd = nd; p.sink = sink;
  p.num_pages = num_pages; p.page_size = page_size; p.num_seqs = num_seqs;
  p.H = H; p.KV = KV; p.G = H / KV; p.Gb = flex_heads_per_block(p.G); p.hparts = p.G / p.Gb;
  p.dk = dk; p.dv = dv; p.dk_pitch = (dk + 63) / 64 * 64;
  p.scale_log2 = scale * LOG2E; p.window = window; p.nsplit = nsplit; p.status = status;
  const long long slabs = (long long)num_items * KV * p.hparts * nsplit;
  p.part_o = scratch;
  p.part_ml = scratch ? scratch + slabs * FLEX_M * dv : nullptr;
  const bool own_v = v_cache != nullptr;
  const int block_n = p.dk_pitch > 256 ? 32 : 64;        // the two key stages and the queries share 227 KB
  const int dvb = dv > 64 ? 128 : 64;
  const int dslices = (dv + dvb - 1) / dvb;
  // items of at most 16 rows (max_rows, 0: unknown) over keys that are their own values: the four warps take a value
  // slice each instead of 16 rows each
  p.warps_are_slices = (!own_v && dslices > 1 && max_rows > 0 && max_rows <= 16) ? 1 : 0;
  const int zblocks = p.warps_are_slices ? (dslices + 3) / 4 : dslices;
  size_t smem = ((size_t)(FLEX_M + 2 * block_n) * p.dk_pitch + (own_v ? (size_t)2 * block_n * dvb : 0)) * sizeof(bf16);
  if (smem > 227 * 1024) return -2;
  const size_t bias_bytes = (size_t)2 * (block_n + FLEX_M / p.Gb) * p.Gb * sizeof(float);
  p.bias_in_smem = dist_bias && smem + bias_bytes <= 227 * 1024 ? 1 : 0;       // else each score fetches its own
  if (p.bias_in_smem) smem += bias_bytes;
  int rc;
  // items of at most 16 rows otherwise: the four warps take a quarter of each tile's keys (tiles of 64 keys only)
  const bool ksplit = !p.warps_are_slices && block_n == 64 && max_rows > 0 && max_rows <= 16;
  if (ksplit) rc = dvb == 128 ? flex_launch<64, 128, 4>(p, zblocks, smem, stream) : flex_launch<64, 64, 4>(p, zblocks, smem, stream);
  else if (block_n == 64) rc = dvb == 128 ? flex_launch<64, 128, 1>(p, zblocks, smem, stream) : flex_launch<64, 64, 1>(p, zblocks, smem, stream);
  else rc = dvb == 128 ? flex_launch<32, 128, 1>(p, zblocks, smem, stream) : flex_launch<32, 64, 1>(p, zblocks, smem, stream);
  if (rc) return rc;
  if (nsplit > 1) {
    attn_flex_merge_kernel<<<dim3(num_items, KV * p.hparts, FLEX_M), 128, 0, stream>>>(p);
  }
  return si_last_error();
}
