// nn.SpatialConvolutionFFTTiled on the native side: the FFT convolution on tiles of the image.
//
// Mirrors the reference's tiled module (fbcunn/SpatialConvolutionFFTTiled.lua:265-365 for the
// constructor, :489-563 / :601-683 / :724-802 for the three passes): the output is cut into
// disjoint tiles of (tile - k + 1) pixels, each of which depends on an input tile of `tile`
// pixels (overlap-save), so the transform size stays at the tile size whatever the image
// size -- which also lifts the 128-pixel limit of the untiled module.
//
// The tiles of one image are extra batch entries of one untiled pass:
//     updateOutput        input tiles (overlapping)   -> output tiles (disjoint)
//     updateGradInput     gradOutput tiles (disjoint) -> gradInput tiles, overlap-added
//     accGradParameters   the contraction's sum over the batch is also the sum over tiles
// Cutting, assembling and the overlap-add are the three small kernels below (each element
// is gathered, so the result does not depend on timing); the tile buffers belong to the
// tiled handle.
#include <cstdio>

#include "../../include/fbfftconv.h"
#include "kernels.h"

using namespace fbfft;

namespace {

struct TileGeom {
  int B, C;            // images, planes of the tensor being cut / assembled
  int H, W;            // extent of the image tensor
  int th, tw;          // extent of one tile
  int sh, sw;          // step between tile origins
  int nh, nw;          // tiles per image
  int oy, ox;          // image coordinate of tile (0, 0)'s first element (negative = padding)
};

// tiles[(b, ty, tx)][c][y][x] = image[b][c][ty*sh + y + oy][tx*sw + x + ox], zero outside the image.
// One block per (tile, plane): the tile's place is worked out once, the threads walk its pixels.
__global__ void __launch_bounds__(128) tiles_cut_kernel(const float* __restrict__ image, float* __restrict__ tiles,
                                                        const __grid_constant__ TileGeom g) {
  const long long planes = (long long)g.B * g.nh * g.nw * g.C;
  const int per_plane = g.th * g.tw;
  for (long long pl = blockIdx.x; pl < planes; pl += gridDim.x) {
    const int c = (int)(pl % g.C);
    const long long tile = pl / g.C;
    const int tx = (int)(tile % g.nw);
    const long long rest = tile / g.nw;
    const int ty = (int)(rest % g.nh);
    const long long b = rest / g.nh;
    const int y0 = ty * g.sh + g.oy, x0 = tx * g.sw + g.ox;
    const float* src = image + (b * g.C + c) * (long long)g.H * g.W;
    float* dst = tiles + pl * per_plane;
    for (int i = threadIdx.x; i < per_plane; i += blockDim.x) {
      const int y = i / g.tw, x = i - y * g.tw;
      const int Y = y0 + y, X = x0 + x;
      dst[i] = (Y >= 0 && Y < g.H && X >= 0 && X < g.W) ? src[Y * g.W + X] : 0.f;
    }
  }
}

// image[b][c][Y][X] = sum over the tiles that cover (Y, X) of their element there (+ bias[c]).
// Disjoint tiles (step = extent) have exactly one; overlapping ones (gradInput) up to
// ceil(th/sh) * ceil(tw/sw).  Image coordinates as in tiles_cut_kernel.  One block per image plane.
__global__ void __launch_bounds__(256) tiles_gather_kernel(const float* __restrict__ tiles, float* __restrict__ image,
                                                           const float* __restrict__ bias,
                                                           const __grid_constant__ TileGeom g) {
  const long long planes = (long long)g.B * g.C;
  const int per_plane = g.H * g.W;
  const int tile_elems = g.th * g.tw;
  for (long long pl = blockIdx.x; pl < planes; pl += gridDim.x) {
    const int c = (int)(pl % g.C);
    const long long b = pl / g.C;
    const float add = bias ? bias[c] : 0.f;
    // tile (ty, tx) of this image and plane starts at base + ((ty*nw + tx)*C) * tile_elems
    const float* base = tiles + (b * g.nh * g.nw * g.C + c) * (long long)tile_elems;
    const long long tile_stride = (long long)g.C * tile_elems;
    float* dst = image + pl * per_plane;
    for (int i = threadIdx.x; i < per_plane; i += blockDim.x) {
      const int Y = i / g.W, X = i - Y * g.W;
      const int py = Y - g.oy, px = X - g.ox;  // position in the tiled (padded) frame, >= 0
      int ty1 = py / g.sh;                      // tiles ty with ty*sh <= py < ty*sh + th
      if (ty1 > g.nh - 1) ty1 = g.nh - 1;
      int tx1 = px / g.sw;
      if (tx1 > g.nw - 1) tx1 = g.nw - 1;
      float acc = add;
      for (int ty = ty1; ty >= 0 && py - ty * g.sh < g.th; --ty)
        for (int tx = tx1; tx >= 0 && px - tx * g.sw < g.tw; --tx)
          acc += base[(ty * g.nw + tx) * tile_stride + (py - ty * g.sh) * g.tw + (px - tx * g.sw)];
      dst[i] = acc;
    }
  }
}

cudaError_t launch_cut(const float* image, float* tiles, const TileGeom& g, cudaStream_t s) {
  const long long planes = (long long)g.B * g.nh * g.nw * g.C;
  const long long cap = (long long)sm_count() * 64;
  tiles_cut_kernel<<<(int)(planes < cap ? planes : cap), 128, 0, s>>>(image, tiles, g);
  count_launch();
  return cudaGetLastError();
}
cudaError_t launch_gather(const float* tiles, float* image, const float* bias, const TileGeom& g, cudaStream_t s) {
  const long long planes = (long long)g.B * g.C;
  const long long cap = (long long)sm_count() * 32;
  tiles_gather_kernel<<<(int)(planes < cap ? planes : cap), 256, 0, s>>>(tiles, image, bias, g);
  count_launch();
  return cudaGetLastError();
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

}  // namespace

struct fbfftconv_tiled {
  fbfftconv_desc d;        // the caller's layer
  fbfftconv_handle* inner; // untiled layer of the tiles: batch * tiles images of th x tw, no padding
  int device;
  int oH, oW;              // output extent of the layer
  int th, tw, sh, sw, nh, nw;
  float* in_tiles = nullptr;   // (B*nh*nw, P, th, tw): input tiles / gradInput tiles
  float* out_tiles = nullptr;  // (B*nh*nw, F, sh, sw): output tiles / gradOutput tiles
};

namespace {

TileGeom input_geom(const fbfftconv_tiled* t) {
  const fbfftconv_desc& d = t->d;
  return TileGeom{d.batch, d.n_input_plane, d.input_h, d.input_w, t->th, t->tw, t->sh, t->sw, t->nh, t->nw, -d.pad_h, -d.pad_w};
}
TileGeom output_geom(const fbfftconv_tiled* t) {
  const fbfftconv_desc& d = t->d;
  return TileGeom{d.batch, d.n_output_plane, t->oH, t->oW, t->sh, t->sw, t->sh, t->sw, t->nh, t->nw, 0, 0};
}

int tiled_fail(int code, const char* message) { return report_error(code, message); }

struct Guard {
  int prev = -1;
  bool switched = false;
  explicit Guard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
  }
  ~Guard() {
    if (switched) cudaSetDevice(prev);
  }
};

int ensure_tiles(fbfftconv_tiled* t) {
  if (t->in_tiles) return FBFFTCONV_OK;
  const size_t tiles = (size_t)t->d.batch * t->nh * t->nw;
  const size_t n_in = tiles * t->d.n_input_plane * t->th * t->tw, n_out = tiles * t->d.n_output_plane * t->sh * t->sw;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (n_in + n_out) * sizeof(float));
  if (e != cudaSuccess) {
    cudaGetLastError();
    char msg[160];
    snprintf(msg, sizeof(msg), "tile buffers of %zu bytes: %s", (n_in + n_out) * sizeof(float), cudaGetErrorString(e));
    return tiled_fail(FBFFTCONV_ERR_NOMEM, msg);
  }
  t->in_tiles = static_cast<float*>(p);
  t->out_tiles = t->in_tiles + n_in;
  return FBFFTCONV_OK;
}

#define TILED_CUDA(expr)                                                          \
  do {                                                                            \
    cudaError_t e_ = (expr);                                                      \
    if (e_ != cudaSuccess) return tiled_fail(FBFFTCONV_ERR_CUDA, cudaGetErrorString(e_)); \
  } while (0)
#define TILED_TRY(expr)                  \
  do {                                   \
    int rc_ = (expr);                    \
    if (rc_ != FBFFTCONV_OK) return rc_; \
  } while (0)

}  // namespace

extern "C" {

int fbfftconv_tiled_create(const fbfftconv_desc* desc, int tile_h, int tile_w, fbfftconv_tiled** out) {
  if (!desc || !out) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  *out = nullptr;
  const fbfftconv_desc& d = *desc;
  if (d.batch <= 0 || d.n_input_plane <= 0 || d.n_output_plane <= 0 || d.input_h <= 0 || d.input_w <= 0 ||
      d.kernel_h <= 0 || d.kernel_w <= 0)
    return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "sizes must be positive");
  if (d.stride_h != 1 || d.stride_w != 1)
    return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "fft only supports stride-1 convolutions");
  if (d.pad_h < 0 || d.pad_w < 0 || d.pad_h >= d.kernel_h || d.pad_w >= d.kernel_w)
    return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "padding must be non-negative and smaller than the kernel");
  if (tile_h <= d.kernel_h - 1 || tile_w <= d.kernel_w - 1)
    return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "tile size must exceed the kernel size minus one");
  const int oH = d.input_h + 2 * d.pad_h - d.kernel_h + 1, oW = d.input_w + 2 * d.pad_w - d.kernel_w + 1;
  if (oH <= 0 || oW <= 0) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "kernel larger than the padded input");
  fbfftconv_tiled* t = new fbfftconv_tiled();
  t->d = d;
  t->oH = oH;
  t->oW = oW;
  t->th = tile_h < d.input_h + 2 * d.pad_h ? tile_h : d.input_h + 2 * d.pad_h;
  t->tw = tile_w < d.input_w + 2 * d.pad_w ? tile_w : d.input_w + 2 * d.pad_w;
  t->sh = t->th - d.kernel_h + 1;  // output tile = step of the input tiles
  t->sw = t->tw - d.kernel_w + 1;
  t->nh = ceil_div(oH, t->sh);
  t->nw = ceil_div(oW, t->sw);
  const long long images = (long long)d.batch * t->nh * t->nw;
  if (images > 65535) {
    delete t;
    return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "batch x tiles per image exceeds 65535: use larger tiles");
  }
  fbfftconv_desc inner = d;
  inner.batch = (int)images;
  inner.input_h = t->th;
  inner.input_w = t->tw;
  inner.pad_h = inner.pad_w = 0;
  const int rc = fbfftconv_create(&inner, &t->inner);
  if (rc != FBFFTCONV_OK) {
    delete t;
    return rc;
  }
  t->device = d.device;
  if (t->device < 0 && cudaGetDevice(&t->device) != cudaSuccess) {
    cudaGetLastError();
    t->device = 0;
  }
  *out = t;
  return FBFFTCONV_OK;
}

int fbfftconv_tiled_destroy(fbfftconv_tiled* t) {
  if (!t) return FBFFTCONV_OK;
  {
    Guard g(t->device);
    if (t->in_tiles) cudaFree(t->in_tiles);
  }
  fbfftconv_destroy(t->inner);
  delete t;
  return FBFFTCONV_OK;
}

fbfftconv_handle* fbfftconv_tiled_inner(fbfftconv_tiled* t) { return t ? t->inner : nullptr; }

size_t fbfftconv_tiled_workspace_bytes(const fbfftconv_tiled* t) {
  if (!t) return 0;
  const size_t tiles = (size_t)t->d.batch * t->nh * t->nw;
  return fbfftconv_workspace_bytes(t->inner) +
         tiles * ((size_t)t->d.n_input_plane * t->th * t->tw + (size_t)t->d.n_output_plane * t->sh * t->sw) * sizeof(float);
}

int fbfftconv_tiled_geometry(const fbfftconv_tiled* t, int32_t out[6]) {
  if (!t || !out) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  out[0] = t->th;
  out[1] = t->tw;
  out[2] = t->sh;
  out[3] = t->sw;
  out[4] = t->nh;
  out[5] = t->nw;
  return FBFFTCONV_OK;
}

int fbfftconv_tiled_update_output(fbfftconv_tiled* t, const float* input, const float* weight, const float* bias,
                                  float* output, fbfftconv_stream stream) {
  if (!t || !input || !weight || !output) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  Guard g(t->device);
  TILED_TRY(validate_device_pointer(t->device, input, "input"));
  TILED_TRY(validate_device_pointer(t->device, bias, "bias"));
  TILED_TRY(validate_device_pointer(t->device, output, "output"));
  TILED_TRY(ensure_tiles(t));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TILED_CUDA(launch_cut(input, t->in_tiles, input_geom(t), s));
  TILED_TRY(fbfftconv_update_output(t->inner, t->in_tiles, weight, nullptr, t->out_tiles, stream));
  // the bias goes on once, while the tiles are put together (fbcunn/SpatialConvolutionFFTTiled.lua:541-544)
  TILED_CUDA(launch_gather(t->out_tiles, output, bias, output_geom(t), s));
  return FBFFTCONV_OK;
}

int fbfftconv_tiled_update_grad_input(fbfftconv_tiled* t, const float* grad_output, const float* weight,
                                      float* grad_input, fbfftconv_stream stream) {
  if (!t || !grad_output || !weight || !grad_input) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  Guard g(t->device);
  TILED_TRY(validate_device_pointer(t->device, grad_output, "gradOutput"));
  TILED_TRY(validate_device_pointer(t->device, grad_input, "gradInput"));
  TILED_TRY(ensure_tiles(t));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TILED_CUDA(launch_cut(grad_output, t->out_tiles, output_geom(t), s));
  TILED_TRY(fbfftconv_update_grad_input(t->inner, t->out_tiles, weight, t->in_tiles, stream));
  TILED_CUDA(launch_gather(t->in_tiles, grad_input, nullptr, input_geom(t), s));  // overlap-add
  return FBFFTCONV_OK;
}

int fbfftconv_tiled_acc_grad_parameters(fbfftconv_tiled* t, const float* input, const float* grad_output,
                                        float* grad_weight, float* grad_bias, float scale, fbfftconv_stream stream) {
  if (!t || !input || !grad_output || !grad_weight) return tiled_fail(FBFFTCONV_ERR_INVALID_ARGUMENT, "null argument");
  Guard g(t->device);
  TILED_TRY(validate_device_pointer(t->device, input, "input"));
  TILED_TRY(validate_device_pointer(t->device, grad_output, "gradOutput"));
  TILED_TRY(ensure_tiles(t));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  TILED_CUDA(launch_cut(input, t->in_tiles, input_geom(t), s));
  TILED_CUDA(launch_cut(grad_output, t->out_tiles, output_geom(t), s));
  return fbfftconv_acc_grad_parameters(t->inner, t->in_tiles, t->out_tiles, grad_weight, grad_bias, scale, stream);
}

}  // extern "C"
