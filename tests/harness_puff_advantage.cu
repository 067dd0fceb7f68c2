// Standalone harness for the advantage op, in the style of the reference's
// tests/test_c_advantage.cu (a plain nvcc program: cudaMalloc'd float buffers,
// one launch, copy back) but for the operator that exists: it calls the C ABI
// of include/puff_advantage.h and compares with a host loop of the recurrence
// (pufferlib/extensions/pufferlib.cpp:28-41).  Exit code 0 = all variants agree.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -o harness tests/harness_puff_advantage.cu \
//        -Lpufferlib_b200 -lpuff_advantage_sm100 -Xlinker -rpath=$PWD/pufferlib_b200
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../include/puff_advantage.h"

static void host_rows(const float* v, const float* r, const float* d, const float* w, float* a, float gamma,
                      float lambda, float rho_clip, float c_clip, int S, int H)
{
    for (int s = 0; s < S; ++s) {
        float last = 0.0f;
        for (int t = H - 2; t >= 0; --t) {
            const long o = (long)s * H;
            const float nn = (float)(1.0 - (double)d[o + t + 1]);
            const float rho = fminf(w[o + t], rho_clip), c = fminf(w[o + t], c_clip);
            const float gv = gamma * v[o + t + 1];
            const float gvn = gv * nn;
            const float td = (r[o + t + 1] + gvn) - v[o + t];
            const float delta = rho * td;
            const float gl = gamma * lambda;
            const float glc = gl * c;
            const float x = glc * last;
            last = delta + x * nn;
            a[o + t] = last;
        }
    }
}

static unsigned lcg(unsigned* s) { return *s = *s * 1664525u + 1013904223u; }
static float unit(unsigned* s) { return (lcg(s) >> 8) * (1.0f / 16777216.0f); }

static int run_case(int S, int H, int variant, const char* name)
{
    const size_t n = (size_t)S * H;
    float *hv = (float*)malloc(n * 4), *hr = (float*)malloc(n * 4), *hd = (float*)malloc(n * 4),
          *hw = (float*)malloc(n * 4), *ha = (float*)malloc(n * 4), *want = (float*)malloc(n * 4);
    unsigned seed = 12345u + S * 31 + H;
    for (size_t i = 0; i < n; ++i) {
        hv[i] = 2.0f * unit(&seed) - 1.0f;
        hr[i] = 0.2f * unit(&seed) - 0.1f;
        hd[i] = unit(&seed) < 0.02f ? 1.0f : 0.0f;
        hw[i] = 0.8f + 0.4f * unit(&seed);
        ha[i] = want[i] = 777.0f;
    }
    host_rows(hv, hr, hd, hw, want, 0.99f, 0.95f, 1.0f, 1.0f, S, H);
    float *dv, *dr, *dd, *dw, *da;
    cudaMalloc(&dv, n * 4); cudaMalloc(&dr, n * 4); cudaMalloc(&dd, n * 4); cudaMalloc(&dw, n * 4); cudaMalloc(&da, n * 4);
    cudaMemcpy(dv, hv, n * 4, cudaMemcpyHostToDevice); cudaMemcpy(dr, hr, n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(dd, hd, n * 4, cudaMemcpyHostToDevice); cudaMemcpy(dw, hw, n * 4, cudaMemcpyHostToDevice);
    cudaMemcpy(da, ha, n * 4, cudaMemcpyHostToDevice);
    const int rc = puff_advantage_sm100_launch(dv, dr, dd, dw, da, NULL, 0.99f, 0.95f, 1.0f, 1.0f, S, H, variant, NULL);
    if (rc != 0) { printf("%s: launch failed: %s\n", name, puff_advantage_sm100_strerror(rc)); return 1; }
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("%s: sync failed\n", name); return 1; }
    cudaMemcpy(ha, da, n * 4, cudaMemcpyDeviceToHost);
    int bad = 0;
    for (size_t i = 0; i < n; ++i) {
        if (variant == PUFF_VARIANT_SCAN) {
            const float tol = fmaxf(1e-6f, 1e-5f * fabsf(want[i]));
            if (!(fabsf(ha[i] - want[i]) <= tol)) ++bad;
        } else if (memcmp(&ha[i], &want[i], 4) != 0) {
            ++bad;
        }
    }
    printf("%s S=%d H=%d kernel=%d mismatches=%d\n", name, S, H, puff_advantage_sm100_last_kernel(), bad);
    cudaFree(dv); cudaFree(dr); cudaFree(dd); cudaFree(dw); cudaFree(da);
    free(hv); free(hr); free(hd); free(hw); free(ha); free(want);
    return bad != 0;
}

int main(void)
{
    int fail = 0;
    fail |= run_case(6, 4, PUFF_VARIANT_SERIAL, "tiny");          // the shape of the reference's stale harness
    fail |= run_case(1000, 64, PUFF_VARIANT_SERIAL, "serial");
    fail |= run_case(333, 91, PUFF_VARIANT_SERIAL, "odd");
    fail |= run_case(40, 2048, PUFF_VARIANT_SCAN, "scan");
    fail |= run_case(77, 50, PUFF_VARIANT_GENERIC, "generic");
    printf(fail ? "FAILED\n" : "OK\n");
    return fail;
}
