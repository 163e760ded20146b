/*
 * CPU ORACLE -- TEST INFRASTRUCTURE ONLY.
 *
 * Restates, with fp64 accumulation, the direct (spatial-domain) definition of the
 * three passes of the FFT convolution module.  It is the checker the CUDA path is
 * compared with; nothing in the product path may link, load or call it.
 *
 * What it follows in the reference (paths relative to the reference checkout):
 *   update_output        test/ReferenceConvolutions.cpp:85-200   (crossCorrelationValidOnly)
 *                        + bias add  src/ConvolutionBias.cu:39-51
 *   update_grad_input    test/ReferenceConvolutions.cpp:338-450  (convolutionFull)
 *   acc_grad_weight      test/ReferenceConvolutions.cpp:452-554  (crossCorrelationReverseValidOnly)
 *   acc_grad_bias        src/ConvolutionBias.cu:61-97  (gradBias[f] = scale * sum gradOutput[:,f,:,:])
 *
 * Differences from that code, on purpose: stride is fixed at 1 (the FFT module
 * asserts it, fbcunn/SpatialConvolutionFBFFT.lua:60-61), padding is symmetric
 * (fbcunn/SpatialConvolutionFFT.lua:171-174), sums are carried in double, and the
 * loops are written in gather form per result plane so that single planes of a
 * large problem can be checked.  Pinned against the compiled reference file and
 * the reference's known-answer test by tests/test_oracle.py.
 *
 * Layouts: input (B,P,iH,iW), weight (F,P,kH,kW), output / gradOutput (B,F,oH,oW)
 * with oH = iH + 2 padH - kH + 1, all contiguous, fp32 in, fp64 out.
 */
#include <stddef.h>
#include <stdint.h>

typedef struct {
  int64_t B, P, F, iH, iW, kH, kW, padH, padW;
} oracle_shape;

static int64_t out_h(const oracle_shape* s) { return s->iH + 2 * s->padH - s->kH + 1; }
static int64_t out_w(const oracle_shape* s) { return s->iW + 2 * s->padW - s->kW + 1; }

/* output[b,f,y,x] = bias[f] + sum_{p,u,v} weight[f,p,u,v] * input[b,p,y+u-padH,x+v-padW] */
static void output_plane(const oracle_shape* s, const float* input, const float* weight,
                         const float* bias, int64_t b, int64_t f, double* dst) {
  const int64_t oH = out_h(s), oW = out_w(s);
  for (int64_t y = 0; y < oH; ++y) {
    for (int64_t x = 0; x < oW; ++x) {
      double acc = 0.0;
      for (int64_t p = 0; p < s->P; ++p) {
        const float* in = input + (b * s->P + p) * s->iH * s->iW;
        const float* w = weight + (f * s->P + p) * s->kH * s->kW;
        for (int64_t u = 0; u < s->kH; ++u) {
          const int64_t iy = y + u - s->padH;
          if (iy < 0 || iy >= s->iH) continue;
          for (int64_t v = 0; v < s->kW; ++v) {
            const int64_t ix = x + v - s->padW;
            if (ix < 0 || ix >= s->iW) continue;
            acc += (double)w[u * s->kW + v] * (double)in[iy * s->iW + ix];
          }
        }
      }
      dst[y * oW + x] = acc + (bias ? (double)bias[f] : 0.0);
    }
  }
}

/* gradInput[b,p,iy,ix] = sum_{f,u,v} weight[f,p,u,v] * gradOutput[b,f,iy+padH-u,ix+padW-v] */
static void grad_input_plane(const oracle_shape* s, const float* grad_output,
                             const float* weight, int64_t b, int64_t p, double* dst) {
  const int64_t oH = out_h(s), oW = out_w(s);
  for (int64_t iy = 0; iy < s->iH; ++iy) {
    for (int64_t ix = 0; ix < s->iW; ++ix) {
      double acc = 0.0;
      for (int64_t f = 0; f < s->F; ++f) {
        const float* go = grad_output + (b * s->F + f) * oH * oW;
        const float* w = weight + (f * s->P + p) * s->kH * s->kW;
        for (int64_t u = 0; u < s->kH; ++u) {
          const int64_t oy = iy + s->padH - u;
          if (oy < 0 || oy >= oH) continue;
          for (int64_t v = 0; v < s->kW; ++v) {
            const int64_t ox = ix + s->padW - v;
            if (ox < 0 || ox >= oW) continue;
            acc += (double)w[u * s->kW + v] * (double)go[oy * oW + ox];
          }
        }
      }
      dst[iy * s->iW + ix] = acc;
    }
  }
}

/* gradWeight[f,p,u,v] = scale * sum_{b,y,x} gradOutput[b,f,y,x] * input[b,p,y+u-padH,x+v-padW] */
static void grad_weight_plane(const oracle_shape* s, const float* input,
                              const float* grad_output, double scale, int64_t f, int64_t p,
                              double* dst) {
  const int64_t oH = out_h(s), oW = out_w(s);
  for (int64_t u = 0; u < s->kH; ++u) {
    for (int64_t v = 0; v < s->kW; ++v) {
      double acc = 0.0;
      for (int64_t b = 0; b < s->B; ++b) {
        const float* in = input + (b * s->P + p) * s->iH * s->iW;
        const float* go = grad_output + (b * s->F + f) * oH * oW;
        for (int64_t y = 0; y < oH; ++y) {
          const int64_t iy = y + u - s->padH;
          if (iy < 0 || iy >= s->iH) continue;
          for (int64_t x = 0; x < oW; ++x) {
            const int64_t ix = x + v - s->padW;
            if (ix < 0 || ix >= s->iW) continue;
            acc += (double)go[y * oW + x] * (double)in[iy * s->iW + ix];
          }
        }
      }
      dst[u * s->kW + v] = scale * acc;
    }
  }
}

static int valid(const oracle_shape* s) {
  return s && s->B > 0 && s->P > 0 && s->F > 0 && s->kH > 0 && s->kW > 0 && s->padH >= 0 &&
         s->padW >= 0 && out_h(s) > 0 && out_w(s) > 0;
}

/* ---- whole tensors -------------------------------------------------------- */

int oracle_update_output(const oracle_shape* s, const float* input, const float* weight,
                         const float* bias, double* output) {
  if (!valid(s)) return 1;
  const int64_t plane = out_h(s) * out_w(s), n = s->B * s->F;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    output_plane(s, input, weight, bias, i / s->F, i % s->F, output + i * plane);
  return 0;
}

int oracle_update_grad_input(const oracle_shape* s, const float* grad_output,
                             const float* weight, double* grad_input) {
  if (!valid(s)) return 1;
  const int64_t plane = s->iH * s->iW, n = s->B * s->P;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    grad_input_plane(s, grad_output, weight, i / s->P, i % s->P, grad_input + i * plane);
  return 0;
}

int oracle_acc_grad_weight(const oracle_shape* s, const float* input, const float* grad_output,
                           double scale, double* grad_weight) {
  if (!valid(s)) return 1;
  const int64_t plane = s->kH * s->kW, n = s->F * s->P;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    grad_weight_plane(s, input, grad_output, scale, i / s->P, i % s->P, grad_weight + i * plane);
  return 0;
}

int oracle_acc_grad_bias(const oracle_shape* s, const float* grad_output, double scale,
                         double* grad_bias) {
  if (!valid(s)) return 1;
  const int64_t plane = out_h(s) * out_w(s);
#pragma omp parallel for schedule(static)
  for (int64_t f = 0; f < s->F; ++f) {
    double acc = 0.0;
    for (int64_t b = 0; b < s->B; ++b) {
      const float* go = grad_output + (b * s->F + f) * plane;
      for (int64_t i = 0; i < plane; ++i) acc += (double)go[i];
    }
    grad_bias[f] = scale * acc;
  }
  return 0;
}

/* ---- selected planes of a large problem ------------------------------------
 * `first[i]`, `second[i]` name plane i: (b,f) for the output, (b,p) for gradInput,
 * (f,p) for gradWeight.  dst holds n planes back to back. */

int oracle_update_output_planes(const oracle_shape* s, const float* input, const float* weight,
                                const float* bias, int64_t n, const int64_t* first,
                                const int64_t* second, double* dst) {
  if (!valid(s)) return 1;
  const int64_t plane = out_h(s) * out_w(s);
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    output_plane(s, input, weight, bias, first[i], second[i], dst + i * plane);
  return 0;
}

int oracle_update_grad_input_planes(const oracle_shape* s, const float* grad_output,
                                    const float* weight, int64_t n, const int64_t* first,
                                    const int64_t* second, double* dst) {
  if (!valid(s)) return 1;
  const int64_t plane = s->iH * s->iW;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    grad_input_plane(s, grad_output, weight, first[i], second[i], dst + i * plane);
  return 0;
}

int oracle_acc_grad_weight_planes(const oracle_shape* s, const float* input,
                                  const float* grad_output, double scale, int64_t n,
                                  const int64_t* first, const int64_t* second, double* dst) {
  if (!valid(s)) return 1;
  const int64_t plane = s->kH * s->kW;
#pragma omp parallel for schedule(dynamic, 1)
  for (int64_t i = 0; i < n; ++i)
    grad_weight_plane(s, input, grad_output, scale, first[i], second[i], dst + i * plane);
  return 0;
}
