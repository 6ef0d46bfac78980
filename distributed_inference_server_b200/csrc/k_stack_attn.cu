// k_stack_attn.cu -- grouped-query attention over paged keys and values for the layer-list decoders (DIS_MIX_ATTENTION and the
// attention half of DIS_MIX_PARALLEL): the per-token preparation (biases, whole-projection query/key norm, partial rotary with a
// frequency table, cache write of the rotated keys and of the values -- own projection or the unrotated keys, optionally
// rotated by their position) and the attention itself with softmax or per-head sigmoid weights, over the whole history or a
// slice of it.  Scores, weights, norms and angles are fp32 (angles are formed in double) whatever the cache's element type.
#include "stack_dev.cuh"

namespace dis {

// ------------------------------------------------------------------------------------------------ preparation
// One block per token.  proj row: queries at q_off [H][d], keys at k_off [G][d], values at v_off [G][dv] (unless values are
// the keys).  `bias` (or null): [H*d + G*d] for q | k, added here when the product left it out.
template <bool F32>
__global__ void __launch_bounds__(128) stack_attn_prep_kernel(const float *proj, long long ld, int q_off, int k_off, int v_off,
                                                              const float *bias, const float *qn, const float *kn, const double *freq,
                                                              const double *vfreq, StackAttn c, StackSpans sp, float *qf, void *kpool,
                                                              void *vpool, float *vrot, const int *page_table, int max_pages,
                                                              int page_size) {
  extern __shared__ float tab[];  // cos [half], sin [half], value cos [dv/2], value sin [dv/2]
  __shared__ float sh[32];
  const int t = blockIdx.x;
  const float *row = proj + (long long)t * ld;
  const int pos = sp.pos[t], slot = sp.slot[t];
  const int half = c.rot_dims >> 1, vhalf = c.dv >> 1;
  const bool rot_v = (c.flags & DIS_ATTN_ROT_V) != 0;
  float *cs = tab, *sn = tab + half, *vcs = sn + half, *vsn = vcs + vhalf;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s_, c_;
    sincos((double)pos * freq[i], &s_, &c_);
    cs[i] = (float)c_; sn[i] = (float)s_;
  }
  if (rot_v)
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
      double s_, c_;
      sincos((double)pos * vfreq[i], &s_, &c_);
      vcs[i] = (float)c_; vsn[i] = (float)s_;
      vrot[(long long)t * c.dv + i] = (float)c_;
      vrot[(long long)t * c.dv + vhalf + i] = (float)s_;
    }
  const int nq = c.H * c.d, nk = c.G * c.d;
  const float *qb = bias, *kb = bias ? bias + nq : nullptr;
  float rq = 1.f, rk = 1.f;
  if (c.flags & DIS_ATTN_QK_NORM) {
    float s = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = row[q_off + i] + (qb ? qb[i] : 0.f); s += v * v; }
    rq = rsqrtf(block_sum(s, sh) / (float)nq + c.eps);
    s = 0.f;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = row[k_off + i] + (kb ? kb[i] : 0.f); s += v * v; }
    rk = rsqrtf(block_sum(s, sh) / (float)nk + c.eps);
  }
  __syncthreads();
  auto val = [&](int off, const float *b, const float *g, float r, int i) {
    float v = row[off + i] + (b ? b[i] : 0.f);
    if (g) v = v * r * g[i];
    return v;
  };
  auto rotated = [&](int off, const float *b, const float *g, float r, int i) {
    const int e = i % c.d;
    if (e >= c.rot_dims) return val(off, b, g, r, i);
    if (e < half) return val(off, b, g, r, i) * cs[e] - val(off, b, g, r, i + half) * sn[e];
    return val(off, b, g, r, i) * cs[e - half] + val(off, b, g, r, i - half) * sn[e - half];
  };
  const float *qg = (c.flags & DIS_ATTN_QK_NORM) ? qn : nullptr, *kg = (c.flags & DIS_ATTN_QK_NORM) ? kn : nullptr;
  for (int i = threadIdx.x; i < nq; i += blockDim.x) qf[(long long)t * nq + i] = rotated(q_off, qb, qg, rq, i);
  const long long prow = (long long)page_table[(long long)slot * max_pages + pos / page_size] * page_size + pos % page_size;
  for (int i = threadIdx.x; i < nk; i += blockDim.x) st_el<F32>(kpool, prow * nk + i, rotated(k_off, kb, kg, rk, i));
  const int nv = c.G * c.dv;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v;
    if (c.flags & DIS_ATTN_V_IS_K) v = row[k_off + i] + (kb ? kb[i] : 0.f);  // dv == d: the keys as projected
    else if (!rot_v) v = row[v_off + i];
    else {
      const int e = i % c.dv;
      v = e < vhalf ? row[v_off + i] * vcs[e] - row[v_off + i + vhalf] * vsn[e]
                    : row[v_off + i] * vcs[e - vhalf] + row[v_off + i - vhalf] * vsn[e - vhalf];
    }
    st_el<F32>(vpool, prow * nv + i, v);
  }
}
cudaError_t launch_stack_attn_prep(const float *proj, long long ld, int q_off, int k_off, int v_off, const float *bias, const float *qn,
                                   const float *kn, const double *freq, const double *vfreq, const StackAttn &c, const StackSpans &sp,
                                   float *qf, void *kpool, void *vpool, float *vrot, bool f32, const int *page_table, int max_pages,
                                   int page_size, cudaStream_t st) {
  if (sp.T <= 0) return cudaSuccess;
  const size_t sh = (size_t)(c.rot_dims + c.dv) * sizeof(float);
  if (f32) stack_attn_prep_kernel<true><<<sp.T, 128, sh, st>>>(proj, ld, q_off, k_off, v_off, bias, qn, kn, freq, vfreq, c, sp, qf, kpool, vpool, vrot, page_table, max_pages, page_size);
  else stack_attn_prep_kernel<false><<<sp.T, 128, sh, st>>>(proj, ld, q_off, k_off, v_off, bias, qn, kn, freq, vfreq, c, sp, qf, kpool, vpool, vrot, page_table, max_pages, page_size);
  return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ attention, fp32 arithmetic
// One CTA per (query block, key/value head, slice of the history).  The block's (token, query head of the group) pairs share
// 32-key tiles staged in shared memory as fp32; one warp per pair at a time: a lane scores one key, then lanes own value
// coordinates.  SIG: weight = sigmoid(score * temp[h] + pb[h]), plain sums.  Otherwise an online softmax (running maximum and
// denominator per pair).  Epilogue (whole history in one CTA) or merge kernel (slices): normalise, rotate the output back by
// the query's position when values were rotated, scale, and store into the mixer's output row.
constexpr int kAtTile = 32, kAtWarps = 8, kAtMaxSplit = 64;

struct AttnOut {
  void *out;          // [T][ld] in the compute type; head h at columns off + h * dv
  long long ld;
  int off;
  float scale;        // factor on the output (weight of this mixer inside a parallel layer)
  const float *vrot;  // [T][dv]: cos | sin of the query position's value angles, or null
};

template <bool F32>
__device__ __forceinline__ void attn_store(const AttnOut &o, const float *a, float inv, int tok, int h, int dv, int j) {
  float v = a[j] * inv;
  if (o.vrot) {  // rotation by minus the angle: (u, v) -> (u cos + v sin, v cos - u sin)
    const int hf = dv >> 1;
    const float *cs = o.vrot + (long long)tok * dv, *sn = cs + hf;
    v = j < hf ? (a[j] * cs[j] + a[j + hf] * sn[j]) * inv : (a[j] * cs[j - hf] - a[j - hf] * sn[j - hf]) * inv;
  }
  st_el<F32>(o.out, (long long)tok * o.ld + o.off + (long long)h * dv + j, v * o.scale);
}

int stack_attn_block_tokens(const StackAttn &c) {
  const int R = c.H / c.G;
  int bq = std::max(1, 32 / R);
  while (bq > 1 && ((size_t)kAtTile * (c.d + c.dv + 2 + kAtWarps) + (size_t)bq * R * (c.d + c.dv + 2)) * 4 > 200 * 1024) bq >>= 1;
  return bq;
}
static size_t attn_smem(const StackAttn &c, int bq) {
  const int R = c.H / c.G;
  return ((size_t)kAtTile * (c.d + c.dv + 2 + kAtWarps) + (size_t)bq * R * (c.d + c.dv + 2)) * sizeof(float);
}

template <bool F32, bool SIG>
__global__ void __launch_bounds__(kAtWarps * 32) stack_attn_kernel(const float *qf, const void *kpool, const void *vpool, const float *temp,
                                                                   const float *pb, StackAttn c, StackSpans sp, const int *qb_tok0,
                                                                   const int *qb_len, const int *page_table, int max_pages,
                                                                   int page_size, AttnOut o, int keys_per_split, float *part) {
  extern __shared__ float shm[];
  const int d = c.d, dv = c.dv, DP = d + 1, VP = dv + 1, R = c.H / c.G, g = blockIdx.y;
  const int tok0 = qb_tok0[blockIdx.x], nq = qb_len[blockIdx.x];
  const int pairs = nq * R;
  float *kt = shm;                               // [32][DP]
  float *vt = kt + (size_t)kAtTile * DP;         // [32][VP]
  float *qs = vt + (size_t)kAtTile * VP;         // [pairs][d]
  float *acc = qs + (size_t)pairs * d;           // [pairs][dv]
  float *mx = acc + (size_t)pairs * dv;          // [pairs]
  float *dn = mx + pairs;                        // [pairs]
  float *prs = dn + pairs;                       // [warps][32]
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  const int slot = sp.slot[tok0];
  const int last_pos = sp.pos[tok0 + nq - 1];
  for (int i = threadIdx.x; i < pairs * d; i += blockDim.x) {
    const int p = i / d, e = i - p * d;
    qs[i] = qf[((long long)(tok0 + p / R) * c.H + g * R + p % R) * d + e];
  }
  for (int i = threadIdx.x; i < pairs * dv; i += blockDim.x) acc[i] = 0.f;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) { mx[i] = -INFINITY; dn[i] = 0.f; }
  const int *pt = page_table + (long long)slot * max_pages;
  const int k_begin = part ? (int)blockIdx.z * keys_per_split : 0;
  const int k_end = part ? min(last_pos + 1, k_begin + keys_per_split) : last_pos + 1;
  const long long krow = (long long)c.G * d, vrow = (long long)c.G * dv;
  for (int k0 = k_begin; k0 < k_end; k0 += kAtTile) {
    const int nk = min(kAtTile, k_end - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < nk * d; i += blockDim.x) {
      const int kk = i / d, cc = i - kk * d, kp = k0 + kk;
      const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
      kt[(size_t)kk * DP + cc] = ld_el<F32>(kpool, prow * krow + (long long)g * d + cc);
    }
    for (int i = threadIdx.x; i < nk * dv; i += blockDim.x) {
      const int kk = i / dv, cc = i - kk * dv, kp = k0 + kk;
      const long long prow = (long long)pt[kp / page_size] * page_size + kp % page_size;
      vt[(size_t)kk * VP + cc] = ld_el<F32>(vpool, prow * vrow + (long long)g * dv + cc);
    }
    __syncthreads();
    for (int p = w; p < pairs; p += kAtWarps) {
      const int qpos = sp.pos[tok0 + p / R], h = g * R + p % R;
      const float *q = qs + (size_t)p * d;
      float sc = -INFINITY;
      if (l < nk && k0 + l <= qpos) {
        const float *kr = kt + (size_t)l * DP;
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;  // four chains, added at the end: the sum's order is fixed by d alone
        int i = 0;
        for (; i + 3 < d; i += 4) {
          s0 = fmaf(q[i], kr[i], s0); s1 = fmaf(q[i + 1], kr[i + 1], s1);
          s2 = fmaf(q[i + 2], kr[i + 2], s2); s3 = fmaf(q[i + 3], kr[i + 3], s3);
        }
        for (; i < d; i++) s0 = fmaf(q[i], kr[i], s0);
        sc = ((s0 + s1) + (s2 + s3)) * c.scale;
      }
      float pr, corr = 1.f, psum = 0.f, m_new = 0.f;
      if (SIG) {
        pr = sc == -INFINITY ? 0.f : 1.f / (1.f + expf(-(sc * temp[h] + pb[h])));
      } else {
        const float m_old = mx[p];
        m_new = fmaxf(m_old, warp_max(sc));
        pr = sc == -INFINITY ? 0.f : expf(sc - m_new);
        corr = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
        psum = warp_sum(pr);
      }
      float *a = acc + (size_t)p * dv;
      float *pw = prs + w * kAtTile;  // the tile's weights of this pair: lanes own coordinates below, so every lane reads all
      pw[l] = pr;
      __syncwarp();
      for (int j = l; j < dv; j += 32) {
        float v0 = a[j] * corr, v1 = 0.f, v2 = 0.f, v3 = 0.f;
        int kk = 0;
        for (; kk + 3 < nk; kk += 4) {
          v0 = fmaf(pw[kk], vt[(size_t)kk * VP + j], v0); v1 = fmaf(pw[kk + 1], vt[(size_t)(kk + 1) * VP + j], v1);
          v2 = fmaf(pw[kk + 2], vt[(size_t)(kk + 2) * VP + j], v2); v3 = fmaf(pw[kk + 3], vt[(size_t)(kk + 3) * VP + j], v3);
        }
        for (; kk < nk; kk++) v0 = fmaf(pw[kk], vt[(size_t)kk * VP + j], v0);
        a[j] = (v0 + v1) + (v2 + v3);
      }
      __syncwarp();
      if (!SIG && l == 0) { mx[p] = m_new; dn[p] = dn[p] * corr + psum; }
      __syncwarp();
    }
  }
  __syncthreads();
  if (!part) {
    for (int i = threadIdx.x; i < pairs * dv; i += blockDim.x) {
      const int p = i / dv, j = i - p * dv;
      attn_store<F32>(o, acc + (size_t)p * dv, SIG ? 1.f : 1.f / dn[p], tok0 + p / R, g * R + p % R, dv, j);
    }
    return;
  }
  // slice record per (token, head): dv unnormalised sums, then the slice's maximum and denominator
  for (int i = threadIdx.x; i < pairs * (dv + 2); i += blockDim.x) {
    const int p = i / (dv + 2), j = i - p * (dv + 2);
    float *rec = part + (((long long)blockIdx.z * sp.T + tok0 + p / R) * c.H + g * R + p % R) * (dv + 2);
    rec[j] = j < dv ? acc[(size_t)p * dv + j] : j == dv ? mx[p] : dn[p];
  }
}

// Merge of the slices of one (token, head): softmax: out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M); sigmoid: plain sum.
// Slices that lie wholly behind the token (nothing visible) wrote m = -inf, l = 0 and zeros.
template <bool F32, bool SIG>
__global__ void stack_attn_merge_kernel(const float *part, int n_split, int T, int H, int dv, AttnOut o) {
  extern __shared__ float msh[];  // [dv] merged sums, [n_split] factors
  float *a = msh, *ws = msh + dv;
  __shared__ float inv_den;
  const int p = blockIdx.x, tok = p / H, h = p - tok * H;
  const long long stride = (long long)T * H * (dv + 2);
  const float *rec = part + (long long)p * (dv + 2);
  if (!SIG) {
    float M = -INFINITY;
    for (int s = 0; s < n_split; s++) M = fmaxf(M, rec[s * stride + dv]);
    for (int s = threadIdx.x; s < n_split; s += blockDim.x) {
      const float m = rec[s * stride + dv];
      ws[s] = m == -INFINITY ? 0.f : expf(m - M);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float den = 0.f;
      for (int s = 0; s < n_split; s++) den += rec[s * stride + dv + 1] * ws[s];
      inv_den = 1.f / den;
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < n_split; s++) v = SIG ? v + rec[s * stride + j] : fmaf(rec[s * stride + j], ws[s], v);
    a[j] = v;
  }
  __syncthreads();
  for (int j = threadIdx.x; j < dv; j += blockDim.x) attn_store<F32>(o, a, SIG ? 1.f : inv_den, tok, h, dv, j);
}

cudaError_t launch_stack_attn(const float *qf, const void *kpool, const void *vpool, bool f32, const float *temp, const float *pb,
                              const StackAttn &c, const StackSpans &sp, const int *qb_tok0, const int *qb_len, int n_qb, int bq,
                              const int *page_table, int max_pages, int page_size, void *out, long long ld_out, int out_off,
                              float out_scale, const float *vrot, int n_split, int keys_per_split, float *part, cudaStream_t st) {
  if (n_qb <= 0) return cudaSuccess;
  if (n_split <= 1 || !part) { n_split = 1; part = nullptr; }
  if (n_split > kAtMaxSplit) return cudaErrorInvalidValue;
  const bool sig = (c.flags & DIS_ATTN_SIGMOID) != 0;
  const size_t sh = attn_smem(c, bq);
  if (sh > 220 * 1024) return cudaErrorInvalidValue;
  static DeviceOnce once;
  DIS_CUDA_TRY(once.run([&] {
    cudaError_t e = cudaFuncSetAttribute(stack_attn_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_attn_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    return e != cudaSuccess ? e : cudaFuncSetAttribute(stack_attn_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  }));
  const AttnOut o{out, ld_out, out_off, out_scale, (c.flags & DIS_ATTN_ROT_V) ? vrot : nullptr};
  const dim3 grid(n_qb, c.G, n_split);
  const int th = kAtWarps * 32;
#define DIS_ATTN_LAUNCH(F, S) \
  stack_attn_kernel<F, S><<<grid, th, sh, st>>>(qf, kpool, vpool, temp, pb, c, sp, qb_tok0, qb_len, page_table, max_pages, page_size, o, keys_per_split, part)
  if (f32 && sig) DIS_ATTN_LAUNCH(true, true);
  else if (f32) DIS_ATTN_LAUNCH(true, false);
  else if (sig) DIS_ATTN_LAUNCH(false, true);
  else DIS_ATTN_LAUNCH(false, false);
#undef DIS_ATTN_LAUNCH
  if (part) {
    const size_t msh = (size_t)(c.dv + n_split) * sizeof(float);
    const int rows = sp.T * c.H;
    if (f32 && sig) stack_attn_merge_kernel<true, true><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else if (f32) stack_attn_merge_kernel<true, false><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else if (sig) stack_attn_merge_kernel<false, true><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
    else stack_attn_merge_kernel<false, false><<<rows, 64, msh, st>>>(part, n_split, sp.T, c.H, c.dv, o);
  }
  return cudaGetLastError();
}

}  // namespace dis
