/*
 * A plain C caller of the C-ABI: no Python, no torch.  It builds a small
 * attention problem and a small decode problem in host memory, runs them
 * through tf_attn_fwd / tf_decode with device buffers from the CUDA runtime,
 * and compares with straightforward host loops.  Exit code 0 = all good.
 *
 *   nvcc -x cu tests/cabi_smoke.c -Iinclude -Ltilefusion_b200 -ltilefusion_b200 -o cabi_smoke
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>

#include "tilefusion_b200.h"

#define CHECK_CUDA(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %s\n", cudaGetErrorString(e), #x); return 2; } } while (0)
#define CHECK_TF(x) do { int rc = (x); if (rc != TF_OK) { printf("tf error %d: %s\n", rc, tf_last_error()); return 3; } } while (0)

static float frand(unsigned* s) { *s = *s * 1664525u + 1013904223u; return ((*s >> 8) & 0xFFFF) / 65536.0f - 0.5f; }

/* softmax(q k^T * scale) v for one head, fp32 on the 16-bit-rounded inputs */
static void host_attention(const __half* q, const __half* k, const __half* v, int lq, int lk, int d, float scale,
                           float* o, float* lse) {
  float* s = (float*)malloc(sizeof(float) * lk);
  for (int i = 0; i < lq; ++i) {
    float m = -INFINITY;
    for (int j = 0; j < lk; ++j) {
      float acc = 0.f;
      for (int c = 0; c < d; ++c) acc += __half2float(q[i * d + c]) * __half2float(k[j * d + c]);
      s[j] = acc * scale;
      if (s[j] > m) m = s[j];
    }
    float l = 0.f;
    for (int j = 0; j < lk; ++j) { s[j] = expf(s[j] - m); l += s[j]; }
    for (int c = 0; c < d; ++c) {
      float acc = 0.f;
      for (int j = 0; j < lk; ++j) acc += s[j] * __half2float(v[j * d + c]);
      o[i * d + c] = acc / l;
    }
    lse[i] = m + logf(l);
  }
  free(s);
}

static int run_case(int lq, int lk, int d, int decode) {
  const size_t nq = (size_t)lq * d, nk = (size_t)lk * d;
  __half* hq = (__half*)malloc(nq * 2), *hk = (__half*)malloc(nk * 2), *hv = (__half*)malloc(nk * 2);
  __half* ho = (__half*)malloc(nq * 2);
  float* hl = (float*)malloc(sizeof(float) * lq), *ro = (float*)malloc(sizeof(float) * nq), *rl = (float*)malloc(sizeof(float) * lq);
  unsigned seed = 1234u + lq + lk;
  for (size_t i = 0; i < nq; ++i) hq[i] = __float2half(frand(&seed) * 2.f);
  for (size_t i = 0; i < nk; ++i) hk[i] = __float2half(frand(&seed) * 2.f);
  for (size_t i = 0; i < nk; ++i) hv[i] = __float2half(frand(&seed) * 2.f);
  const float scale = 1.0f / sqrtf((float)d);
  host_attention(hq, hk, hv, lq, lk, d, scale, ro, rl);

  void *dq, *dk, *dv, *dout, *dl, *ws = NULL;
  CHECK_CUDA(cudaMalloc(&dq, nq * 2)); CHECK_CUDA(cudaMalloc(&dk, nk * 2)); CHECK_CUDA(cudaMalloc(&dv, nk * 2));
  CHECK_CUDA(cudaMalloc(&dout, nq * 2)); CHECK_CUDA(cudaMalloc(&dl, sizeof(float) * lq));
  CHECK_CUDA(cudaMemcpy(dq, hq, nq * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dk, hk, nk * 2, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dv, hv, nk * 2, cudaMemcpyHostToDevice));
  if (!decode) {
    TfAttnDesc a = {0};
    a.dtype = TF_F16; a.batch = 1; a.heads = 1; a.len_q = lq; a.len_kv = lk; a.head_dim = d; a.head_dim_v = d;
    a.softmax_scale = scale;
    a.q_stride_l = d; a.k_stride_l = d; a.k_stride_d = 1; a.v_stride_l = d; a.v_stride_d = 1; a.o_stride_l = d;
    CHECK_TF(tf_attn_fwd(dq, dk, dv, dout, (float*)dl, &a, NULL));
  } else {
    TfDecodeDesc t = {0};
    TfDecodePlan plan;
    t.dtype = TF_F16; t.batch = 1; t.heads = 1; t.len_kv = lk; t.head_dim = d; t.softmax_scale = scale;
    CHECK_TF(tf_decode_plan(&t, &plan));
    CHECK_CUDA(cudaMalloc(&ws, plan.workspace_bytes));
    CHECK_TF(tf_decode(dq, dk, dv, dout, (float*)dl, ws, plan.workspace_bytes, &t, NULL));
  }
  int code = 0;
  CHECK_TF(tf_device_status(&code));
  CHECK_CUDA(cudaMemcpy(ho, dout, nq * 2, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaMemcpy(hl, dl, sizeof(float) * lq, cudaMemcpyDeviceToHost));
  float max_o = 0.f, max_l = 0.f;
  for (size_t i = 0; i < nq; ++i) { float e = fabsf(__half2float(ho[i]) - ro[i]); if (!(e <= max_o)) max_o = e; }
  for (int i = 0; i < lq; ++i) { float e = fabsf(hl[i] - rl[i]); if (!(e <= max_l)) max_l = e; }
  printf("%s lq=%d lk=%d d=%d: max |dO| = %.2e, max |dLSE| = %.2e\n", decode ? "decode " : "prefill", lq, lk, d, max_o, max_l);
  cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dout); cudaFree(dl); if (ws) cudaFree(ws);
  free(hq); free(hk); free(hv); free(ho); free(hl); free(ro); free(rl);
  return (max_o <= 2e-2f && max_l <= 1e-3f) ? 0 : 1;      /* the tolerances of the Python parity tests */
}

int main(void) {
  if (tf_abi_version() != 5) { printf("unexpected ABI version %d\n", tf_abi_version()); return 4; }
  int bad = 0;
  bad |= run_case(200, 300, 128, 0);
  bad |= run_case(64, 128, 64, 0);
  bad |= run_case(1, 2000, 128, 1);
  printf(bad ? "FAILED\n" : "ok\n");
  return bad;
}
