/*
 * Plain-C restatement of the reference's algorithms for the normalization / softmax path.
 * TEST INFRASTRUCTURE ONLY: used by tests/ (and bench.py's CPU legs) as a checker, never by the
 * product.  All functions work on fp32 arrays with fp32 accumulation, which is what the reference
 * does for fp32 / fp16 / bf16 inputs (acc_type = float); 16-bit storage is handled by the caller
 * (upcast before, round once after).  Citations are paths within intel/torch-xpu-ops.
 *
 * Parity pin: these restatements are checked against PyTorch CPU ATen and against the golden
 * vectors in tests/golden/ (tests/test_oracle.py).  The reference's SYCL sources cannot be built
 * here, so its own binary is not part of the pin.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

/* Welford running moments, one element at a time, then a pairwise merge — the scheme of
 * WelfordOnlineSum / WelfordCombine (src/ATen/native/xpu/sycl/LayerNormKernels.cpp:353-392).  The
 * reference spreads a row over the lanes of a work-group (4 elements per lane per step) and merges
 * lane states; `lanes` reproduces that split (lanes = 1 is the textbook serial form).  Exact
 * division replaces the reference's native reciprocal. */
typedef struct { float mean, m2, count; } moments_t;

static moments_t moments_push(moments_t s, float v) {
  const float delta = v - s.mean;
  s.count += 1.0f;
  s.mean += delta / s.count;
  s.m2 += delta * (v - s.mean);
  return s;
}

static moments_t moments_merge(moments_t a, moments_t b) {
  moments_t r = {0.0f, 0.0f, a.count + b.count};
  if (r.count > 0.0f) {
    const float delta = b.mean - a.mean;
    const float na = a.count / r.count, nb = b.count / r.count;
    r.mean = na * a.mean + nb * b.mean;
    r.m2 = a.m2 + b.m2 + delta * delta * a.count * nb;
  }
  return r;
}

/* layer norm forward: VectorizedLayerNormKernelFunctor (LayerNormKernels.cpp:469-586):
 * rstd = rsqrt(m2 / N + eps); y = gamma * (rstd * (x - mean)) + beta.
 * rms = 1: sigma2 = sum x^2 (:365), rstd = rsqrt(sigma2 / N + eps), y = gamma * (rstd * x). */
void ref_norm_fwd(const float* x, const float* gamma, const float* beta, float* y, float* mean, float* rstd,
                  int64_t M, int64_t N, float eps, int rms, int lanes) {
  if (lanes < 1) lanes = 1;
  for (int64_t i = 0; i < M; ++i) {
    const float* xr = x + i * N;
    float mu = 0.0f, rs;
    if (rms) {
      float s = 0.0f;
      for (int64_t j = 0; j < N; ++j) s += xr[j] * xr[j];
      rs = 1.0f / sqrtf(s / (float)N + eps);
    } else {
      moments_t total = {0.0f, 0.0f, 0.0f};
      for (int l = 0; l < lanes; ++l) {
        moments_t st = {0.0f, 0.0f, 0.0f};
        /* lane l owns 4-element vectors l, l + lanes, l + 2*lanes, ... (:409-416) */
        for (int64_t v = l; v * 4 < N; v += lanes)
          for (int64_t j = v * 4; j < v * 4 + 4 && j < N; ++j) st = moments_push(st, xr[j]);
        total = moments_merge(total, st);
      }
      mu = total.mean;
      rs = 1.0f / sqrtf(total.m2 / (float)N + eps);
    }
    for (int64_t j = 0; j < N; ++j) {
      float t = rs * (xr[j] - mu);
      if (gamma) t *= gamma[j];
      if (!rms && beta) t += beta[j];
      y[i * N + j] = t;
    }
    if (mean && !rms) mean[i] = mu;
    if (rstd) rstd[i] = rs;
  }
}

/* backward w.r.t. x: LayerNormBackward::reduce_combine / update (LayerNormKernels.cpp:96-126,
 * :150-186): sum1 = sum dy*gamma, sum2 = sum dy*gamma*(x-mean)*rstd,
 * dx = (rstd / N) * (N*gamma*dy - (x-mean)*rstd*sum2 - sum1); rms: mean = 0, no sum1. */
void ref_norm_bwd_dx(const float* dy, const float* x, const float* mean, const float* rstd, const float* gamma,
                     float* dx, int64_t M, int64_t N, int rms) {
  for (int64_t i = 0; i < M; ++i) {
    const float mu = rms ? 0.0f : mean[i], rs = rstd[i];
    float sum1 = 0.0f, sum2 = 0.0f;
    for (int64_t j = 0; j < N; ++j) {
      const float g = gamma ? dy[i * N + j] * gamma[j] : dy[i * N + j];
      if (!rms) sum1 += g;
      sum2 += g * (x[i * N + j] - mu) * rs;
    }
    const float term1 = (1.0f / (float)N) * rs;
    for (int64_t j = 0; j < N; ++j) {
      float f = (float)N * (gamma ? gamma[j] * dy[i * N + j] : dy[i * N + j]);
      f -= (x[i * N + j] - mu) * rs * sum2;
      if (!rms) f -= sum1;
      dx[i * N + j] = f * term1;
    }
  }
}

/* weight gradients: GammaBetaBackwardSimpleKernelFunctor (LayerNormKernels.cpp:876-1024):
 * dgamma_j = sum_i dy_ij * (x_ij - mean_i) * rstd_i ; dbeta_j = sum_i dy_ij.  Accumulated in
 * double here so the restatement can also serve as the "fp64 sum" of the reduction gate. */
void ref_norm_bwd_wgrad(const float* dy, const float* x, const float* mean, const float* rstd, double* dgamma,
                        double* dbeta, int64_t M, int64_t N, int rms) {
  for (int64_t j = 0; j < N; ++j) {
    if (dgamma) dgamma[j] = 0.0;
    if (dbeta) dbeta[j] = 0.0;
  }
  for (int64_t i = 0; i < M; ++i) {
    const double mu = rms ? 0.0 : (double)mean[i], rs = (double)rstd[i];
    for (int64_t j = 0; j < N; ++j) {
      const double d = (double)dy[i * N + j];
      if (dgamma) dgamma[j] += d * ((double)x[i * N + j] - mu) * rs;
      if (dbeta && !rms) dbeta[j] += d;
    }
  }
}

/* softmax / log-softmax over dim of an [outer, N, inner] tensor: the three passes of
 * SoftmaxForwardKernelFunctor (src/ATen/native/xpu/sycl/SoftMaxKernels.cpp:546-684): max starts
 * at the lowest finite value (:566-577), sum of exp(x - max) (:583-592), then exp(x-max)/sum or
 * x - max - log(sum) (:611-664). */
void ref_softmax_fwd(const float* x, float* y, int64_t outer, int64_t N, int64_t inner, int is_log) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t in = 0; in < inner; ++in) {
      const float* xp = x + o * N * inner + in;
      float* yp = y + o * N * inner + in;
      float mx = -3.402823466e+38f;
      for (int64_t j = 0; j < N; ++j) mx = fmaxf(mx, xp[j * inner]);
      float s = 0.0f;
      for (int64_t j = 0; j < N; ++j) s += expf(xp[j * inner] - mx);
      const float lg = logf(s);
      for (int64_t j = 0; j < N; ++j) {
        const float d = xp[j * inner] - mx;
        yp[j * inner] = is_log ? d - lg : expf(d) / s;
      }
    }
}

/* backward: SoftmaxBackwardKernelFunctor (SoftMaxKernels.cpp:1229-1347):
 * softmax dx = y * (dy - sum y*dy); log-softmax dx = dy - exp(y) * sum dy. */
void ref_softmax_bwd(const float* dy, const float* y, float* dx, int64_t outer, int64_t N, int64_t inner,
                     int is_log) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t in = 0; in < inner; ++in) {
      const int64_t base = o * N * inner + in;
      float s = 0.0f;
      for (int64_t j = 0; j < N; ++j)
        s += is_log ? dy[base + j * inner] : dy[base + j * inner] * y[base + j * inner];
      for (int64_t j = 0; j < N; ++j) {
        const float d = dy[base + j * inner], yy = y[base + j * inner];
        dx[base + j * inner] = is_log ? d - expf(yy) * s : yy * (d - s);
      }
    }
}

/* nll_loss forward, 2-D input with a reduction: NllLossForwardReduce2DKernelFunctor
 * (src/ATen/native/xpu/sycl/LossNLLKernel.cpp:142-226): out = sum_i -w[t_i]*x[i,t_i],
 * total_weight = sum_i w[t_i], rows with t == ignore_index skipped, mean divides by total_weight.
 * Returns -1 when a target is out of range (the reference asserts on the device, :30-35). */
int ref_nll_fwd(const float* logp, const int64_t* target, const float* weight, float* out, float* total_weight,
                int64_t M, int64_t C, int reduction_mean, int64_t ignore_index) {
  float s = 0.0f, ws = 0.0f;
  for (int64_t i = 0; i < M; ++i) {
    const int64_t t = target[i];
    if (t == ignore_index) continue;
    if (t < 0 || t >= C) return -1;
    const float w = weight ? weight[t] : 1.0f;
    s -= w * logp[i * C + t];
    ws += w;
  }
  *total_weight = ws;
  *out = reduction_mean ? s / ws : s;
  return 0;
}
