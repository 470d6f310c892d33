// K0: objective gradients on the device, per-class |g|/|h| maxima, quantize + pack + root sums.
// Parity: src/objective/cuda/cuda_binary_objective.cu:L132-168, cuda_multiclass_objective.cu:L15-83,
// cuda_regression_objective.cu:L60-476, cuda_rank_objective.cu:L26-194 (one block per query),
// src/treelearner/cuda/cuda_gradient_discretizer.cu:L18-337 (min/max reduce, Philox stochastic
// rounding, packing), cuda_leaf_splits.cu:L19-288 (root sums).
// Differences on purpose: no host synchronisation anywhere (scales stay in device scalars); the
// stochastic rounding is keyed on the GLOBAL row id so a model does not depend on the GPU count;
// lambdarank computes every pair from both documents' threads, so there are no floating-point
// atomics and the gradients are deterministic.
#include "kernels.cuh"

namespace fb {

namespace {

__device__ inline float AtomicMaxPositive(float* addr, float v) {
  // non-negative floats order like their bit patterns
  return __uint_as_float(atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v)));
}

__device__ inline void BlockMax2(float a, float b, float* out2) {
  __shared__ float sa[32], sb[32];
  for (int o = 16; o > 0; o >>= 1) { a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o)); b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o)); }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sa[w] = a; sb[w] = b; }
  __syncthreads();
  if (w == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    a = l < nw ? sa[l] : 0.f; b = l < nw ? sb[l] : 0.f;
    for (int o = 16; o > 0; o >>= 1) { a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, o)); b = fmaxf(b, __shfl_xor_sync(0xffffffffu, b, o)); }
    if (l == 0) { AtomicMaxPositive(out2, a); AtomicMaxPositive(out2 + 1, b); }
  }
}

__device__ inline float SignF(float x) { return (x > 0.f) - (x < 0.f); }

// Pointwise objectives: one thread per row, all classes of the row for multiclass.
__global__ void PointwiseGradKernel(ObjDesc d, const float* __restrict__ score, const float* __restrict__ label, const float* __restrict__ weight,
                                    int n, float* __restrict__ grad, float* __restrict__ hess, float* __restrict__ maxbuf) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float mg = 0.f, mh = 0.f;
  const int K = d.kind == kObjMulticlass ? d.num_class : 1;
  if (i < n) {
    const float w = weight ? weight[i] : 1.f;
    const float y = label[i];
    if (d.kind == kObjMulticlass) {
      float mx = score[i];
      for (int c = 1; c < K; ++c) mx = fmaxf(mx, score[static_cast<size_t>(c) * n + i]);
      float sum = 0.f;
      for (int c = 0; c < K; ++c) sum += expf(score[static_cast<size_t>(c) * n + i] - mx);
      const int yi = static_cast<int>(y);
      const float factor = static_cast<float>(K) / (K - 1.f);
      for (int c = 0; c < K; ++c) {
        const float p = expf(score[static_cast<size_t>(c) * n + i] - mx) / sum;
        const float g = (p - (yi == c ? 1.f : 0.f)) * w, h = factor * p * (1.f - p) * w;
        grad[static_cast<size_t>(c) * n + i] = g; hess[static_cast<size_t>(c) * n + i] = h;
      }
    } else {
      const float s = score[i];
      float g, h;
      switch (d.kind) {
        case kObjBinary: {
          const bool pos = y > 0.f; const float yy = pos ? 1.f : -1.f, sig = static_cast<float>(d.p0);
          const float lw = (pos ? static_cast<float>(d.p2) : static_cast<float>(d.p1)) * w;
          const float r = -yy * sig / (1.f + expf(yy * sig * s)), ar = fabsf(r);
          g = r * lw; h = ar * (sig - ar) * lw; break;
        }
        case kObjL2: g = (s - y) * w; h = w; break;
        case kObjL1: g = SignF(s - y) * w; h = w; break;
        case kObjHuber: { const float df = s - y, a = static_cast<float>(d.p0); g = (fabsf(df) <= a ? df : SignF(df) * a) * w; h = w; break; }
        case kObjFair: { const float x = s - y, c = static_cast<float>(d.p0), dd = fabsf(x) + c; g = c * x / dd * w; h = c * c / (dd * dd) * w; break; }
        case kObjPoisson: { const float e = expf(s); g = (e - y) * w; h = e * expf(static_cast<float>(d.p0)) * w; break; }
        case kObjQuantile: { const float a = static_cast<float>(d.p0); g = ((s - y) >= 0.f ? (1.f - a) : -a) * w; h = w; break; }
        case kObjGamma: { const float e = expf(-s); g = (1.f - y * e) * w; h = y * e * w; break; }
        case kObjTweedie: { const float rho = static_cast<float>(d.p0), e1 = expf((1.f - rho) * s), e2 = expf((2.f - rho) * s); g = (-y * e1 + e2) * w; h = (-y * (1.f - rho) * e1 + (2.f - rho) * e2) * w; break; }
        case kObjXent: { const float z = 1.f / (1.f + expf(-s)); g = (z - y) * w; h = z * (1.f - z) * w; break; }
        case kObjMape: g = SignF(s - y) * (w / fmaxf(1.f, fabsf(y))); h = w; break;   // the label weight 1 / max(1, |y|) scales the gradient only
        case kObjXentLambda: {
          // cross entropy with the weight inside the link: z = 1 - exp(-w log(1 + e^s)); evaluated in double, as the host objective does
          const double wd = w, yd = y, epf = exp(static_cast<double>(s)), hhat = log1p(epf);
          const double z = 1.0 - exp(-wd * hhat), enf = 1.0 / epf;
          g = static_cast<float>((1.0 - yd / z) * wd / (1.0 + enf));
          const double c = 1.0 / (1.0 - z), dd = 1.0 + epf, a = wd * epf / (dd * dd), b = (c / ((c - 1.0) * (c - 1.0))) * (1.0 + wd * epf - c);
          h = static_cast<float>(a * (1.0 + yd * b));
          break;
        }
        default: g = 0.f; h = 0.f;
      }
      grad[i] = g; hess[i] = h;
    }
  }
  // maxima are per class: a second pass over this thread's own values keeps the code simple
  for (int c = 0; c < K; ++c) {
    mg = (i < n) ? fabsf(grad[static_cast<size_t>(c) * n + i]) : 0.f;
    mh = (i < n) ? fabsf(hess[static_cast<size_t>(c) * n + i]) : 0.f;
    BlockMax2(mg, mh, maxbuf + 2 * c);
    __syncthreads();
  }
}

// Several L2 targets (multi_regression): target c of row i has its label at [c][i]; one tree per target and round.
__global__ void MultiRegGradKernel(const float* __restrict__ score, const float* __restrict__ label, const float* __restrict__ weight, int n,
                                   float* __restrict__ grad, float* __restrict__ hess, float* __restrict__ maxbuf) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y;
  float g = 0.f, h = 0.f;
  if (i < n) {
    const float w = weight ? weight[i] : 1.f;
    const size_t o = static_cast<size_t>(c) * n + i;
    g = (score[o] - label[o]) * w; h = w;
    grad[o] = g; hess[o] = h;
  }
  BlockMax2(fabsf(g), fabsf(h), maxbuf + 2 * c);
}

// OVA: class c is a binary problem "label == c".
__global__ void OvaGradKernel(ObjDesc d, const float* __restrict__ score, const float* __restrict__ label, const float* __restrict__ weight, int n,
                              float* __restrict__ grad, float* __restrict__ hess, float* __restrict__ maxbuf) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y;
  float g = 0.f, h = 0.f;
  if (i < n) {
    const float w = weight ? weight[i] : 1.f, sig = static_cast<float>(d.p0);
    const float yy = static_cast<int>(label[i]) == c ? 1.f : -1.f;
    const float r = -yy * sig / (1.f + expf(yy * sig * score[static_cast<size_t>(c) * n + i])), ar = fabsf(r);
    g = r * w; h = ar * (sig - ar) * w;
    grad[static_cast<size_t>(c) * n + i] = g; hess[static_cast<size_t>(c) * n + i] = h;
  }
  BlockMax2(fabsf(g), fabsf(h), maxbuf + 2 * c);
}

// Custom gradients: only the maxima are needed.
__global__ void AbsMaxKernel(const float* __restrict__ grad, const float* __restrict__ hess, int n, float* __restrict__ maxbuf,
                             const uint8_t* __restrict__ mask) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int c = blockIdx.y;
  const bool in = i < n && (mask == nullptr || mask[i] != 0);   // out-of-bag rows do not set the scale
  float g = in ? fabsf(grad[static_cast<size_t>(c) * n + i]) : 0.f, h = in ? fabsf(hess[static_cast<size_t>(c) * n + i]) : 0.f;
  BlockMax2(g, h, maxbuf + 2 * c);
}

// XE-NDCG (rank_xendcg): one block per query. rho = softmax of the query's scores; every document draws gamma from a
// counter-based generator keyed on (row, round, seed), the same draw as the host objective; three passes of block sums
// give the first-, second- and third-order terms of the gradient. Arithmetic in double, as on the host.
// Parity: src/objective/cuda/cuda_rank_objective.cu:L864-981, src/objective/rank_objective.hpp (RankXENDCG).
__device__ inline double BlockSumD(double v, double* scratch) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();                       // scratch may still be read from the previous reduction
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < (blockDim.x >> 5); ++w) t += scratch[w];   // same order in every thread
  return t;
}
__global__ void XendcgKernel(const float* __restrict__ score, const float* __restrict__ label, const float* __restrict__ weight, const int* __restrict__ qb,
                             unsigned int round, unsigned int seed, float* __restrict__ grad, float* __restrict__ hess, float* __restrict__ maxbuf) {
  __shared__ double scratch[32];
  const int q = blockIdx.x;
  const int b = qb[q], cnt = qb[q + 1] - b;
  float mg = 0.f, mh = 0.f;
  if (cnt <= 1) {
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) { grad[b + i] = 0.f; hess[b + i] = 0.f; }
  } else {
    double mx = -1e300;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) mx = fmax(mx, static_cast<double>(score[b + i]));
    for (int o = 16; o > 0; o >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mx;
    __syncthreads();
    for (int w = 0; w < (blockDim.x >> 5); ++w) mx = fmax(mx, scratch[w]);
    double part = 0.0;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) part += exp(static_cast<double>(score[b + i]) - mx);
    const double sum = BlockSumD(part, scratch);
    part = 0.0;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
      const double u = U01From24(Philox4x32_10(static_cast<uint32_t>(b + i), round, 0x1234u, 0x5678u, seed, 0xABCDu).v[0]);
      part += exp2(static_cast<double>(static_cast<int>(label[b + i]))) - u;
    }
    const double inv_denom = 1.0 / fmax(static_cast<double>(kEpsilon), BlockSumD(part, scratch));
    // the per-document terms are recomputed in each pass instead of being kept: queries can be longer than a block
    auto rho_of = [&](int i) { return exp(static_cast<double>(score[b + i]) - mx) / sum; };
    auto l1_of = [&](int i, double rho) {
      const double u = U01From24(Philox4x32_10(static_cast<uint32_t>(b + i), round, 0x1234u, 0x5678u, seed, 0xABCDu).v[0]);
      return -(exp2(static_cast<double>(static_cast<int>(label[b + i]))) - u) * inv_denom + rho;
    };
    part = 0.0;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) { const double rho = rho_of(i); part += l1_of(i, rho) / (1.0 - rho); }
    const double sum_l1 = BlockSumD(part, scratch);
    part = 0.0;
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
      const double rho = rho_of(i); const double p1 = l1_of(i, rho) / (1.0 - rho);
      part += rho * (sum_l1 - p1) / (1.0 - rho);
    }
    const double sum_l2 = BlockSumD(part, scratch);
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) {
      const double rho = rho_of(i); const double l1 = l1_of(i, rho); const double p1 = l1 / (1.0 - rho);
      const double l2 = rho * (sum_l1 - p1); const double p2 = l2 / (1.0 - rho);
      const float w = weight != nullptr ? weight[b + i] : 1.f;
      const float g = static_cast<float>(l1 + l2 + rho * (sum_l2 - p2)) * w, h = static_cast<float>(rho * (1.0 - rho)) * w;
      grad[b + i] = g; hess[b + i] = h;
      mg = fmaxf(mg, fabsf(g)); mh = fmaxf(mh, fabsf(h));
    }
  }
  BlockMax2(mg, mh, maxbuf);
}

// LambdaRank: one block per query, documents ranked by counting (stable, no shared-memory sort
// network), then every document's thread walks all of its pairs.
constexpr int kRankMaxDocs = 2048;
constexpr int kRankMaxLevels = 64;   // label levels counted per query in shared memory (more: the slower scan)
__global__ void LambdarankKernel(const float* __restrict__ score, const float* __restrict__ label, const float* __restrict__ weight,
                                 const int* __restrict__ qb, int num_queries, const double* __restrict__ label_gain, int num_gain, float sigmoid,
                                 int norm, int trunc, float* __restrict__ grad, float* __restrict__ hess, float* __restrict__ maxbuf) {
  extern __shared__ float smem[];
  const int q = blockIdx.x;
  float mg = 0.f, mh = 0.f;
  if (q < num_queries) {
    const int begin = qb[q], cnt = qb[q + 1] - begin;
    float* s_score = smem;                                   // by rank
    float* s_gain = smem + cnt;                              // by rank
    int* s_doc = reinterpret_cast<int*>(smem + 2 * cnt);     // rank -> doc
    float* s_raw = smem + 3 * cnt;                           // by document: the scores, read once from global memory
    float* s_disc = smem + 4 * cnt;                          // by rank: 1 / log2(2 + rank)
    __shared__ float s_red[32];
    __shared__ float s_inv_max_dcg, s_factor;
    __shared__ int s_level_count[kRankMaxLevels];
    for (int i = threadIdx.x; i < cnt; i += blockDim.x) { s_raw[i] = score[begin + i]; s_disc[i] = 1.f / log2f(2.f + i); }
    for (int i = threadIdx.x; i < kRankMaxLevels; i += blockDim.x) s_level_count[i] = 0;
    __syncthreads();
    const bool few_levels = num_gain <= kRankMaxLevels;
    for (int dcur = threadIdx.x; dcur < cnt; dcur += blockDim.x) {
      const float sd = s_raw[dcur];
      int rank = 0;
      for (int o = 0; o < cnt; ++o) { const float so = s_raw[o]; rank += (so > sd) || (so == sd && o < dcur); }
      s_score[rank] = sd; s_doc[rank] = dcur;
      int lab = static_cast<int>(label[begin + dcur]);
      lab = lab < num_gain ? lab : num_gain - 1;
      s_gain[rank] = static_cast<float>(label_gain[lab]);
      if (few_levels) atomicAdd(&s_level_count[lab], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      // ideal DCG at the truncation level: the gains in descending label order, position by position (the same sum,
      // in the same order, as a scan over all documents per label level would give, from the per-level counts)
      double m = 0.0; int pos = 0;
      if (few_levels) {
        for (int lv = num_gain - 1; lv >= 0 && pos < trunc; --lv) {
          const float gv = static_cast<float>(label_gain[lv]);
          for (int k = 0; k < s_level_count[lv] && pos < trunc; ++k) { m += gv / log2(2.0 + pos); ++pos; }
        }
      } else {
        for (int lv = num_gain - 1; lv >= 0 && pos < trunc; --lv) {
          const float gv = static_cast<float>(label_gain[lv]);
          for (int r = 0; r < cnt && pos < trunc; ++r) if (s_gain[r] == gv) { m += gv / log2(2.0 + pos); ++pos; }
        }
      }
      s_inv_max_dcg = m > 0.0 ? static_cast<float>(1.0 / m) : 0.f;
    }
    __syncthreads();
    const float inv = s_inv_max_dcg;
    const float best = s_score[0], worst = s_score[cnt - 1];
    float local_sum = 0.f;
    // pass 1: lambdas of this thread's documents
    for (int p = threadIdx.x; p < cnt; p += blockDim.x) {
      float lg = 0.f, lh = 0.f;
      const float gp = s_gain[p], sp = s_score[p], dp = s_disc[p];
      for (int o = 0; o < cnt; ++o) {
        if (o == p) continue;
        const int lo_rank = o < p ? o : p;
        if (lo_rank >= trunc || lo_rank >= cnt - 1) continue;
        const float go = s_gain[o];
        if (go == gp) continue;
        const bool p_high = gp > go;
        const float ds = p_high ? sp - s_score[o] : s_score[o] - sp;
        const float gap = fabsf(gp - go), pd = fabsf(dp - s_disc[o]);
        float delta = gap * pd * inv;
        if (norm && best != worst) delta /= (0.01f + fabsf(ds));
        const float rho = 1.f / (1.f + expf(sigmoid * ds));
        const float pl = -sigmoid * delta * rho, ph = sigmoid * sigmoid * delta * rho * (1.f - rho);
        lg += p_high ? pl : -pl; lh += ph;
        if (o > p) local_sum -= 2.f * pl;   // each pair counted once
      }
      s_score[p + 0] = s_score[p];   // keep
      grad[begin + s_doc[p]] = lg; hess[begin + s_doc[p]] = lh;
    }
    // block sum of lambdas for the normalisation
    for (int o = 16; o > 0; o >>= 1) local_sum += __shfl_xor_sync(0xffffffffu, local_sum, o);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = local_sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f; for (int w = 0; w < (blockDim.x + 31) / 32; ++w) t += s_red[w];
      s_factor = (norm && t > 0.f) ? log2f(1.f + t) / t : 1.f;
    }
    __syncthreads();
    const float f = s_factor;
    for (int p = threadIdx.x; p < cnt; p += blockDim.x) {
      const int doc = begin + s_doc[p];
      const float w = weight ? weight[doc] : 1.f;
      const float g = grad[doc] * f * w, h = hess[doc] * f * w;
      grad[doc] = g; hess[doc] = h;
      mg = fmaxf(mg, fabsf(g)); mh = fmaxf(mh, fabsf(h));
    }
  }
  __syncthreads();
  BlockMax2(mg, mh, maxbuf);
}

// Quantize one class: packed int16|uint16 words + integer root sums (order-independent).
__global__ void QuantizeKernel(const float* __restrict__ grad, const float* __restrict__ hess, int n, const float* __restrict__ maxbuf,
                               const float* __restrict__ global_max, int bins, int stochastic, uint32_t seed, uint32_t iter_key,
                               unsigned long long global_row_offset, uint8_t* __restrict__ gh_base, int gh_stride, float* __restrict__ scales_out,
                               long long* __restrict__ root_sums, const uint8_t* __restrict__ mask) {
  const float* mx = global_max != nullptr ? global_max : maxbuf;
  float gs = mx[0] / static_cast<float>(bins / 2), hs = mx[1] / static_cast<float>(bins);
  if (!(gs > 0.f)) gs = 1.f;
  if (!(hs > 0.f)) hs = 1.f;
  const float ig = 1.0f / gs, ih = 1.0f / hs;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  long long sg = 0, sh = 0;
  if (i < n) {
    const int32_t w = QuantizeRow(grad[i], hess[i], ig, ih, stochastic != 0, seed, iter_key, global_row_offset + static_cast<unsigned long long>(i));
    *reinterpret_cast<int32_t*>(gh_base + static_cast<size_t>(i) * gh_stride) = w;
    if (mask == nullptr || mask[i] != 0) { sg = UnpackG(w); sh = UnpackH(w); }   // root sums cover the bag only
  }
  for (int o = 16; o > 0; o >>= 1) { sg += __shfl_xor_sync(0xffffffffu, sg, o); sh += __shfl_xor_sync(0xffffffffu, sh, o); }
  __shared__ long long s1[32], s2[32];
  const int wq = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { s1[wq] = sg; s2[wq] = sh; }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long a = 0, b = 0; const int nw = (blockDim.x + 31) >> 5;
    for (int k = 0; k < nw; ++k) { a += s1[k]; b += s2[k]; }
    atomicAdd(reinterpret_cast<unsigned long long*>(root_sums), static_cast<unsigned long long>(a));
    atomicAdd(reinterpret_cast<unsigned long long*>(root_sums + 1), static_cast<unsigned long long>(b));
    if (blockIdx.x == 0) { scales_out[0] = gs; scales_out[1] = hs; }
  }
}

// ---- fixed-point extras: outlier-robust scale and error feedback (shared per-row code in fb/learner.h) ----
// Rows by log-magnitude of the gradient, per block in shared memory, then one global add per non-empty bucket.
__global__ void GradMagHistKernel(const float* __restrict__ grad, int n, const float* __restrict__ max2, const uint8_t* __restrict__ mask,
                                  unsigned long long* __restrict__ hist) {
  __shared__ unsigned int s_hist[kQuantMagBuckets];
  for (int b = threadIdx.x; b < kQuantMagBuckets; b += blockDim.x) s_hist[b] = 0u;
  __syncthreads();
  const float gmax = max2[0];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    if (mask != nullptr && mask[i] == 0) continue;
    const float a = fabsf(grad[i]);
    if (a > 0.f && gmax > 0.f) atomicAdd(&s_hist[QuantMagBucket(a, gmax)], 1u);
  }
  __syncthreads();
  for (int b = threadIdx.x; b < kQuantMagBuckets; b += blockDim.x) { const unsigned int v = s_hist[b]; if (v != 0u) atomicAdd(hist + b, static_cast<unsigned long long>(v)); }
}
// One thread: the gate. qmax = (gradient magnitude of the top level, hessian maximum); clamp = levels at which the
// gradient saturates (0: no saturation, the scale is the plain maximum).
__global__ void RobustScaleKernel(const unsigned long long* __restrict__ hist, long long num_rows, const float* __restrict__ max2, int bins, int use_gate,
                                  float* __restrict__ qmax, int* __restrict__ clamp) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const float gmax = max2[0];
  float top = gmax;
  if (use_gate && gmax > 0.f) top = RobustGradAnchor(hist, num_rows, gmax);
  qmax[0] = top; qmax[1] = max2[1];
  clamp[0] = top < gmax ? bins / 2 : 0;
}
__global__ void QuantizeFeedbackKernel(const float* __restrict__ grad, const float* __restrict__ hess, int n, const float* __restrict__ qmax, const int* __restrict__ clamp,
                                       int bins, int8_t* __restrict__ residual, uint8_t* __restrict__ gh_base, int gh_stride, float* __restrict__ scales_out,
                                       long long* __restrict__ root_sums, const uint8_t* __restrict__ mask) {
  float gs = qmax[0] / static_cast<float>(bins / 2), hs = qmax[1] / static_cast<float>(bins);
  if (!(gs > 0.f)) gs = 1.f;
  if (!(hs > 0.f)) hs = 1.f;
  const float ig = 1.0f / gs, ih = 1.0f / hs;
  const int cl = clamp[0];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  long long sg = 0, sh = 0;
  if (i < n) {
    const bool in_bag = mask == nullptr || mask[i] != 0;
    int8_t* r = (residual != nullptr && in_bag) ? residual + 2 * static_cast<size_t>(i) : nullptr;   // out-of-bag residuals stay
    const int32_t w = QuantizeRowFeedback(grad[i], hess[i], ig, ih, cl, r);
    *reinterpret_cast<int32_t*>(gh_base + static_cast<size_t>(i) * gh_stride) = w;
    if (in_bag) { sg = UnpackG(w); sh = UnpackH(w); }
  }
  for (int o = 16; o > 0; o >>= 1) { sg += __shfl_xor_sync(0xffffffffu, sg, o); sh += __shfl_xor_sync(0xffffffffu, sh, o); }
  __shared__ long long s1[32], s2[32];
  const int wq = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { s1[wq] = sg; s2[wq] = sh; }
  __syncthreads();
  if (threadIdx.x == 0) {
    long long a = 0, b = 0; const int nw = (blockDim.x + 31) >> 5;
    for (int k = 0; k < nw; ++k) { a += s1[k]; b += s2[k]; }
    atomicAdd(reinterpret_cast<unsigned long long*>(root_sums), static_cast<unsigned long long>(a));
    atomicAdd(reinterpret_cast<unsigned long long*>(root_sums + 1), static_cast<unsigned long long>(b));
    if (blockIdx.x == 0) { scales_out[0] = gs; scales_out[1] = hs; }
  }
}

// Full precision: interleave (g, h) and produce per-block partial sums (summed later in a fixed order).
__global__ void InterleaveKernel(const float* __restrict__ grad, const float* __restrict__ hess, int n, float2* __restrict__ gh2,
                                 double* __restrict__ partial /* 2 per block */, const uint8_t* __restrict__ mask) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  double sg = 0, sh = 0;
  if (i < n) { const float g = grad[i], h = hess[i]; gh2[i] = make_float2(g, h); if (mask == nullptr || mask[i] != 0) { sg = g; sh = h; } }
  for (int o = 16; o > 0; o >>= 1) { sg += __shfl_xor_sync(0xffffffffu, sg, o); sh += __shfl_xor_sync(0xffffffffu, sh, o); }
  __shared__ double s1[32], s2[32];
  const int wq = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { s1[wq] = sg; s2[wq] = sh; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0, b = 0; const int nw = (blockDim.x + 31) >> 5;
    for (int k = 0; k < nw; ++k) { a += s1[k]; b += s2[k]; }
    partial[2 * blockIdx.x] = a; partial[2 * blockIdx.x + 1] = b;
  }
}

__global__ void __launch_bounds__(1024) SumPartialsKernel(const double* __restrict__ partial, int nblocks, double* __restrict__ out2) {
  // one block, fixed order: thread t takes blocks t, t+1024, ...; then a fixed shared-memory tree (the same sum on every run)
  __shared__ double sa[1024], sb[1024];
  double a = 0, b = 0;
  for (int k = threadIdx.x; k < nblocks; k += 1024) { a += partial[2 * k]; b += partial[2 * k + 1]; }
  sa[threadIdx.x] = a; sb[threadIdx.x] = b;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) { if (threadIdx.x < o) { sa[threadIdx.x] += sa[threadIdx.x + o]; sb[threadIdx.x] += sb[threadIdx.x + o]; } __syncthreads(); }
  if (threadIdx.x == 0) { out2[0] = sa[0]; out2[1] = sb[0]; }
}

}  // namespace

void LaunchObjectiveGradients(const ObjDesc& d, const float* score, const float* label, const float* weight, const int* qb, int num_queries,
                              const double* label_gain, int num_gain, int n, float* grad, float* hess, float* maxbuf, cudaStream_t s) {
  const int K = (d.kind == kObjMulticlass || d.kind == kObjMulticlassOVA || d.kind == kObjMultiReg) ? d.num_class : 1;
  FB_CUDA(cudaMemsetAsync(maxbuf, 0, sizeof(float) * 2 * K, s));
  const int threads = 256, blocks = (n + threads - 1) / threads;
  if (n <= 0) return;
  if (d.kind == kObjLambdarank) {
    int maxdocs = d.max_docs;
    if (maxdocs > kRankMaxDocs) Log::Fatal("lambdarank on the device supports at most %d documents per query (got %d)", kRankMaxDocs, maxdocs);
    const size_t sm = static_cast<size_t>(maxdocs) * 5 * sizeof(float);
    const int t = maxdocs <= 128 ? 128 : 256;
    LambdarankKernel<<<num_queries, t, sm, s>>>(score, label, weight, qb, num_queries, label_gain, num_gain, static_cast<float>(d.p0), d.p1 != 0.0,
                                               static_cast<int>(d.p2), grad, hess, maxbuf);
  } else if (d.kind == kObjXendcg) {
    XendcgKernel<<<num_queries, 128, 0, s>>>(score, label, weight, qb, static_cast<unsigned int>(d.p1), static_cast<unsigned int>(static_cast<int>(d.p0)), grad, hess, maxbuf);
  } else if (d.kind == kObjMulticlassOVA) {
    OvaGradKernel<<<dim3(blocks, K), threads, 0, s>>>(d, score, label, weight, n, grad, hess, maxbuf);
  } else if (d.kind == kObjMultiReg) {
    MultiRegGradKernel<<<dim3(blocks, K), threads, 0, s>>>(score, label, weight, n, grad, hess, maxbuf);
  } else {
    PointwiseGradKernel<<<blocks, threads, 0, s>>>(d, score, label, weight, n, grad, hess, maxbuf);
  }
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchAbsMax(const float* grad, const float* hess, int n, int num_class, float* maxbuf, cudaStream_t s, const uint8_t* mask) {
  FB_CUDA(cudaMemsetAsync(maxbuf, 0, sizeof(float) * 2 * num_class, s));
  if (n <= 0) return;
  const int threads = 256, blocks = (n + threads - 1) / threads;
  AbsMaxKernel<<<dim3(blocks, num_class), threads, 0, s>>>(grad, hess, n, maxbuf, mask);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchQuantize(const float* grad, const float* hess, int n, const float* maxbuf, const float* global_max, int bins, bool stochastic, uint32_t seed,
                    uint32_t iter_key, uint64_t global_row_offset, uint8_t* gh_base, int gh_stride, float* scales_out, long long* root_sums, cudaStream_t s, const uint8_t* mask) {
  FB_CUDA(cudaMemsetAsync(root_sums, 0, sizeof(long long) * 2, s));
  const int threads = 256, blocks = std::max(1, (n + threads - 1) / threads);
  QuantizeKernel<<<blocks, threads, 0, s>>>(grad, hess, n, maxbuf, global_max, bins, stochastic ? 1 : 0, seed, iter_key, global_row_offset, gh_base, gh_stride, scales_out, root_sums, mask);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchGradMagHist(const float* grad, int n, const float* max2, const uint8_t* mask, unsigned long long* hist, cudaStream_t s) {
  FB_CUDA(cudaMemsetAsync(hist, 0, sizeof(unsigned long long) * kQuantMagBuckets, s));
  if (n <= 0) return;
  const int threads = 256, blocks = std::max(1, std::min(1184, (n + threads * 8 - 1) / (threads * 8)));
  GradMagHistKernel<<<blocks, threads, 0, s>>>(grad, n, max2, mask, hist);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchRobustScale(const unsigned long long* hist, long long num_rows, const float* max2, int bins, bool use_gate, float* qmax, int* clamp, cudaStream_t s) {
  RobustScaleKernel<<<1, 32, 0, s>>>(hist, num_rows, max2, bins, use_gate ? 1 : 0, qmax, clamp);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}
void LaunchQuantizeFeedback(const float* grad, const float* hess, int n, const float* qmax, const int* clamp, int bins, int8_t* residual, uint8_t* gh_base, int gh_stride,
                            float* scales_out, long long* root_sums, cudaStream_t s, const uint8_t* mask) {
  FB_CUDA(cudaMemsetAsync(root_sums, 0, sizeof(long long) * 2, s));
  const int threads = 256, blocks = std::max(1, (n + threads - 1) / threads);
  QuantizeFeedbackKernel<<<blocks, threads, 0, s>>>(grad, hess, n, qmax, clamp, bins, residual, gh_base, gh_stride, scales_out, root_sums, mask);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

void LaunchInterleave(const float* grad, const float* hess, int n, float2* gh2, double* partial, int partial_capacity, double* root_sums_d, cudaStream_t s, const uint8_t* mask) {
  const int threads = 256, blocks = std::max(1, (n + threads - 1) / threads);
  if (blocks > partial_capacity) Log::Fatal("partial-sum buffer too small");
  InterleaveKernel<<<blocks, threads, 0, s>>>(grad, hess, n, gh2, partial, mask);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
  SumPartialsKernel<<<1, 1024, 0, s>>>(partial, blocks, root_sums_d);
  FB_LAUNCHED(); FB_KERNEL_CHECK();
}

}  // namespace fb
