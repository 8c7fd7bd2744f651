// Token sampling from bf16 logits: temperature + optional top-k / top-p support restriction,
// drawn with the Gumbel-max trick and a counter-based Philox4x32-10 generator.
//
//   token = argmax_j ( z_j + G_j ),  z = logit / T,  G_j = -log(-log(u_j)),
//   u_j = word (j mod 4) of Philox(seed; counter = (j div 4, row_key low word, step, row_key high
//   word)), j the global vocab id
// (one Philox4x32 evaluation serves four consecutive ids).
// Every vocabulary id owns its own random number, so the draw does not depend on how the
// vocabulary is sharded over tensor-parallel ranks: each rank reduces its shard to (best value,
// best id) and the global winner is the maximum over ranks (ties -> smaller id).
// Top-k / top-p: a per-row logit threshold `min_keep[row]` (computed by the keep-mask op) removes
// ids whose z is below it; ids at or beyond the real vocab are never sampled.
// kSampleSegs CTAs per row, each reducing a contiguous slice of the row to (best score, best id)
// in a small scratch array; a second kernel picks the winner (maximum, ties to the smaller id --
// an order-free rule, so the split into segments does not change the result).
// Replaces the torch sort/softmax/cumsum path of rl_engine/ops/sampling/policy.py:17-52 for the
// draw itself (FlashInfer sampling in rl_engine/ops/sampling/api.py:42-79).
#include "rlk/host.h"
#include "rlk/ptx.cuh"

namespace rlk {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
  const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
  const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}
__device__ __forceinline__ void philox_4x32(uint64_t seed, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                            uint32_t (&out)[4]) {
  uint32_t c[4] = {c0, c1, c2, c3};
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  out[0] = c[0]; out[1] = c[1]; out[2] = c[2]; out[3] = c[3];
}
__device__ __forceinline__ float gumbel_from_u32(uint32_t r) {
  const float u = (static_cast<float>(r >> 8) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
  return -__logf(-__logf(u));
}

constexpr int kSampleSegs = 8;

struct SampleParams {
  const __nv_bfloat16* logits; long long ld;
  const float* min_keep;       // [rows] or null
  const long long* row_keys;   // [rows] stable per-sequence key for the RNG counter, or null (row index)
  long long* out_ids; float* out_val;
  float* part_val; long long* part_id;   // [rows][kSampleSegs] scratch
  int rows, n_local; long long vocab_start;
  float inv_temp; uint64_t seed; uint32_t step; int greedy;
};

__global__ void __launch_bounds__(256) sample_gumbel_kernel(const SampleParams p) {
  griddep_sync();
  __shared__ float sval[256];
  __shared__ long long sidx[256];
  const int row = blockIdx.x / kSampleSegs, seg = blockIdx.x % kSampleSegs;
  const __nv_bfloat16* src = p.logits + row * p.ld;
  const int nchunks = p.n_local / 8;
  const int per_seg = (nchunks + kSampleSegs - 1) / kSampleSegs;
  const int c_begin = seg * per_seg, c_end = min(nchunks, c_begin + per_seg);
  // 64-bit row key: the low word is the per-sequence / per-position key, the high word may carry
  // anything else that must change the draw (e.g. the training step of a captured decode graph,
  // whose scalar arguments are frozen at capture)
  const unsigned long long rk = static_cast<unsigned long long>(p.row_keys ? p.row_keys[row] : row);
  const uint32_t key = static_cast<uint32_t>(rk), key_hi = static_cast<uint32_t>(rk >> 32);
  const float thr = p.min_keep ? p.min_keep[row] : -INFINITY;
  float best = -INFINITY;
  long long best_id = 0x7fffffffffffffffll;
  uint32_t r4[4] = {0u, 0u, 0u, 0u};
  long long r4_group = -1;          // the four-id group whose random words r4 holds
  for (int c = c_begin + threadIdx.x; c < c_end; c += blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(src + c * 8);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float z = ((k & 1) ? bf16_hi(u[k >> 1]) : bf16_lo(u[k >> 1])) * p.inv_temp;
      if (z < thr) continue;
      const long long id = p.vocab_start + c * 8 + k;
      float s = z;
      if (!p.greedy) {
        const long long grp = id >> 2;
        if (grp != r4_group) {
          philox_4x32(p.seed, static_cast<uint32_t>(grp), key, p.step, key_hi, r4);
          r4_group = grp;
        }
        const int wsel = static_cast<int>(id & 3);
        s += gumbel_from_u32(wsel == 0 ? r4[0] : wsel == 1 ? r4[1] : wsel == 2 ? r4[2] : r4[3]);
      }
      if (s > best || (s == best && id < best_id)) { best = s; best_id = id; }
    }
  }
  sval[threadIdx.x] = best;
  sidx[threadIdx.x] = best_id;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const float ov = sval[threadIdx.x + o];
      const long long oi = sidx[threadIdx.x + o];
      if (ov > sval[threadIdx.x] || (ov == sval[threadIdx.x] && oi < sidx[threadIdx.x])) {
        sval[threadIdx.x] = ov;
        sidx[threadIdx.x] = oi;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    p.part_val[row * kSampleSegs + seg] = sval[0];
    p.part_id[row * kSampleSegs + seg] = sidx[0];
  }
}

__global__ void sample_pick_kernel(const SampleParams p) {
  griddep_sync();
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= p.rows) return;
  float best = p.part_val[row * kSampleSegs];
  long long id = p.part_id[row * kSampleSegs];
  for (int s = 1; s < kSampleSegs; ++s) {
    const float v = p.part_val[row * kSampleSegs + s];
    const long long i = p.part_id[row * kSampleSegs + s];
    if (v > best || (v == best && i < id)) { best = v; id = i; }
  }
  p.out_ids[row] = id;
  if (p.out_val) p.out_val[row] = best;
}

// ------------------------------------------------------------------------------------ top-k / top-p
// Per-row support threshold without sorting.  bf16 logits take at most 65536 distinct values, so
// two 256-bin histogram passes over an order-preserving 16-bit key (high byte, then low byte inside
// the crossing bin) locate the cut exactly:
//   top-k: the k-th largest value (ties with it are all kept, like `z >= kth` in the torch policy);
//   top-p: the smallest value v whose strictly-greater mass is still below top_p * total mass.
// Masses are exp(z - zmax) in 32.32 fixed point summed with integer atomics, so the result does not
// depend on the order in which threads arrive.  (The torch policy walks a stable sort and may cut
// inside a group of equal values; a threshold keeps or drops the whole group -- it keeps it.)
__device__ __forceinline__ uint32_t bf16_order_key(uint32_t h) {  // larger value -> larger key
  return (h & 0x8000u) ? (~h & 0xffffu) : (h | 0x8000u);
}
__device__ __forceinline__ uint32_t bf16_from_order_key(uint32_t k) {
  return (k & 0x8000u) ? (k & 0x7fffu) : (~k & 0xffffu);
}

struct KeepParams {
  const __nv_bfloat16* logits; long long ld;
  int rows, n;
  float inv_temp; int top_k; float top_p;
  float* out_thr;
};

__global__ void __launch_bounds__(512) sample_keep_threshold_kernel(const KeepParams p) {
  __shared__ unsigned int cnt[256];
  __shared__ unsigned long long mass[256];
  __shared__ unsigned int cnt2[256];
  __shared__ unsigned long long mass2[256];
  __shared__ unsigned int red[16];
  __shared__ int s_bk, s_bp;
  __shared__ unsigned int s_cnt_above;
  __shared__ unsigned long long s_mass_above, s_target;
  const int row = blockIdx.x, tid = threadIdx.x;
  const unsigned short* src = reinterpret_cast<const unsigned short*>(p.logits + row * p.ld);
  const bool want_k = p.top_k > 0 && p.top_k < p.n, want_p = p.top_p < 1.f;
  // ---- pass 0: maximum key (NaN never enters: its key compares like a huge value only for +NaN;
  //      logits are finite by contract)
  unsigned int kmax = 0;
  for (int i = tid; i < p.n; i += blockDim.x) kmax = max(kmax, bf16_order_key(src[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) kmax = max(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
  if ((tid & 31) == 0) red[tid >> 5] = kmax;
  if (tid < 256) { cnt[tid] = 0u; mass[tid] = 0ull; cnt2[tid] = 0u; mass2[tid] = 0ull; }
  __syncthreads();
  kmax = 0;
  for (int w = 0; w < 16; ++w) kmax = max(kmax, red[w]);
  const float zmax = __uint_as_float(bf16_from_order_key(kmax) << 16) * p.inv_temp;
  auto weight = [&](uint32_t h) -> unsigned long long {
    const float z = __uint_as_float(h << 16) * p.inv_temp;
    return static_cast<unsigned long long>(__expf(z - zmax) * 4294967296.0f);
  };
  // ---- pass 1: histogram over the high byte of the key
  for (int i = tid; i < p.n; i += blockDim.x) {
    const uint32_t h = src[i], k = bf16_order_key(h);
    atomicAdd(&cnt[k >> 8], 1u);
    if (want_p) atomicAdd(&mass[k >> 8], weight(h));
  }
  __syncthreads();
  if (tid == 0) {
    unsigned int c = 0;
    int bk = 0;
    if (want_k) {
      for (int b = 255; b >= 0; --b) {
        if (c + cnt[b] >= static_cast<unsigned int>(p.top_k)) { bk = b; break; }
        c += cnt[b];
      }
    }
    s_bk = bk;
    s_cnt_above = c;
    unsigned long long total = 0ull, m = 0ull;
    int bp = 0;
    if (want_p) {
      for (int b = 0; b < 256; ++b) total += mass[b];
      const unsigned long long target = static_cast<unsigned long long>(static_cast<double>(p.top_p) * static_cast<double>(total));
      for (int b = 255; b >= 0; --b) {
        // the cut lies in the first non-empty bin (from the top) whose end reaches the target
        if (mass[b] != 0ull && m + mass[b] >= target) { bp = b; break; }
        m += mass[b];
      }
      s_target = target;
    }
    s_bp = bp;
    s_mass_above = m;
  }
  __syncthreads();
  // ---- pass 2: histograms over the low byte inside the crossing bins
  const uint32_t bk = s_bk, bp = s_bp;
  for (int i = tid; i < p.n; i += blockDim.x) {
    const uint32_t h = src[i], k = bf16_order_key(h);
    if (want_k && (k >> 8) == bk) atomicAdd(&cnt2[k & 255u], 1u);
    if (want_p && (k >> 8) == bp) atomicAdd(&mass2[k & 255u], weight(h));
  }
  __syncthreads();
  if (tid == 0) {
    float thr = -INFINITY;
    if (want_k) {
      unsigned int c = s_cnt_above;
      uint32_t key = bk << 8;
      for (int b = 255; b >= 0; --b) {
        c += cnt2[b];
        if (c >= static_cast<unsigned int>(p.top_k)) { key = (bk << 8) | b; break; }
      }
      thr = fmaxf(thr, __uint_as_float(bf16_from_order_key(key) << 16) * p.inv_temp);
    }
    if (want_p) {
      unsigned long long m = s_mass_above;
      uint32_t key = bp << 8;
      // descending: a value is kept while the mass strictly above it is below the target; the
      // row maximum (nothing above it) is always kept
      for (int b = 255; b >= 0; --b) {
        if (mass2[b] == 0ull) continue;
        if (m >= s_target && m != 0ull) break;
        key = (bp << 8) | b;
        m += mass2[b];
      }
      thr = fmaxf(thr, __uint_as_float(bf16_from_order_key(key) << 16) * p.inv_temp);
    }
    p.out_thr[row] = thr;
  }
}

}  // namespace rlk
using namespace rlk;

// out_ids[row] = sampled GLOBAL vocab id from this shard's columns; out_val = its perturbed score
// (the cross-rank winner is the shard with the largest out_val, ties to the smaller id).
// scratch: rows * 8 floats followed by rows * 8 int64 (see rlk_sample_scratch_bytes).
RLK_API long long rlk_sample_scratch_bytes(int rows) { return static_cast<long long>(rows) * kSampleSegs * 12; }

RLK_API int rlk_sample_gumbel(const void* logits, long long ld, const float* min_keep,
                              const long long* row_keys, long long* out_ids, float* out_val,
                              void* scratch, int rows,
                              int n_local, long long vocab_start, float inv_temp,
                              unsigned long long seed, unsigned int step, int greedy, void* stream) {
  RLK_REQUIRE(rows > 0 && n_local > 0 && n_local % 8 == 0 && ld % 8 == 0, "sample: bad shape");
  RLK_REQUIRE(scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 7) == 0, "sample: scratch required (8-byte aligned)");
  long long* part_id = static_cast<long long*>(scratch);
  float* part_val = reinterpret_cast<float*>(part_id + static_cast<long long>(rows) * kSampleSegs);
  SampleParams p{(const __nv_bfloat16*)logits, ld, min_keep, row_keys, out_ids, out_val, part_val, part_id,
                 rows, n_local, vocab_start, inv_temp, seed, step, greedy};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RLK_CHECK_CUDA(launch_pdl(sample_gumbel_kernel, dim3(rows * kSampleSegs), dim3(256), 0, s, p));
  RLK_CHECK_CUDA(launch_pdl(sample_pick_kernel, dim3((rows + 127) / 128), dim3(128), 0, s, p));
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}

// out_thr[row] = smallest scaled logit (logit * inv_temp) that stays in the sampling support under
// top-k (0 = off) and top-p (1 = off); -inf when neither cuts.  Feed it to rlk_sample_gumbel as
// `min_keep`.  One CTA per row, three passes over the row (L2 resident).
RLK_API int rlk_sample_keep_threshold(const void* logits, long long ld, int rows, int n, float inv_temp,
                                      int top_k, float top_p, float* out_thr, void* stream) {
  RLK_REQUIRE(rows > 0 && n > 0, "sample_keep_threshold: empty");
  RLK_REQUIRE(top_p > 0.f, "sample_keep_threshold: top_p must be positive");
  KeepParams p{(const __nv_bfloat16*)logits, ld, rows, n, inv_temp, top_k, top_p, out_thr};
  sample_keep_threshold_kernel<<<rows, 512, 0, static_cast<cudaStream_t>(stream)>>>(p);
  RLK_CHECK_CUDA(cudaGetLastError());
  return RLK_OK;
}
