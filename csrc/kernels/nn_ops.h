// C ABI of the training-op kernels (NHWC bf16 activations, fp32 parameters and
// statistics).  Same calling conventions as kernels.h.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct GeepsConvGeom {
  int B, H, W, C;       // input tensor [B][H][W][C]
  int c0, Cg;           // channel group [c0, c0+Cg) taken by this call
  int KH, KW, stride, pad, OH, OW;
  int ldcol;            // row pitch of the patch matrix, >= KH*KW*Cg, multiple of 8
} GeepsConvGeom;

typedef struct GeepsPoolGeom {
  int B, H, W, C, K, stride, pad, OH, OW;
  int ldx, ldy;         // channel pitch of input / output pixels (>= C; concat slices)
} GeepsPoolGeom;

int geeps_nchw_f32_to_nhwc_bf16(const float* x, void* y, int B, int C, int H, int W, int Cpad, void* stream);
// NCHW (fp32, or bf16 when x_is_bf16) -> NHWC bf16 with the channels zero-padded to Cpad
int geeps_nchw_to_nhwc_bf16(const void* x, int x_is_bf16, void* y, int B, int C, int H, int W, int Cpad, void* stream);
// NCHW (fp32 or bf16) -> space-to-depth NHWC bf16 [B][Hs][Ws][Cpad], channel (dy*S + dx)*C + c, zero-padded
int geeps_nchw_to_s2d_bf16(const void* x, int x_is_bf16, void* y, int B, int C, int H, int W, int S, int Hs, int Ws,
                           int Cpad, void* stream);
// Data transformer: uint8 NCHW source images [B][C][Hin][Win] -> bf16 activations of the H x W crop, as NHWC
// [B][Hs = H][Ws = W][Cpad] (S <= 1) or in the space-to-depth layout [B][Hs][Ws][Cpad] (S > 1); every value becomes
// (pixel - mean[c]) * scale, channels past S*S*C and positions past the crop are zero.  aug: NULL (centre crop, no
// mirror) or 3 ints per image on the device: {h_off, w_off, mirror}.  C <= 4.
typedef struct GeepsU8Transform {
  const unsigned char* x;
  void* y;
  const int* aug;
  int B, C, Hin, Win, H, W, S, Hs, Ws, Cpad;
  float mean[4];
  float scale;
} GeepsU8Transform;
int geeps_u8_transform_bf16(const GeepsU8Transform* p, void* stream);
// g[r][c] = 0 where mask[c] == 0 (fp32 matrix, pitch ld)
int geeps_col_mask_f32(float* g, const unsigned char* mask, long long rows, int cols, long long ld, void* stream);
int geeps_im2col(const void* x, void* col, const GeepsConvGeom* g, void* stream);
int geeps_col2im(const void* dcol, void* dx, const GeepsConvGeom* g, int accumulate, void* stream);

// sums: 2*C floats of scratch; mean_rstd: 2*C floats saved for backward.
int geeps_bn_forward(const void* x, void* y, const float* gamma, const float* beta, float* sums,
                     float* mean_rstd, float* running_mean, float* running_var, long long P, int C,
                     long long ldx, long long ldy, float eps, float momentum, int relu, void* stream);
int geeps_bn_backward(const void* x, const void* dy, const void* y, void* dx, const float* mean_rstd,
                      const float* gamma, float* sums, float* dgamma, float* dbeta, long long P, int C,
                      long long ldx, long long lddy, long long lddx, int relu, float grad_scale, void* stream);
// Training-loop forms: `sums` (2 C floats) must be zero on entry; `zero_after` (2 C floats or NULL) is zeroed for the
// layer's next reduction; the statistics are finalised inside the normalising kernel.  Two launches each, or - with
// `barrier` (4 ints, zero at first use, private to this layer and direction) - ONE cooperative launch whose blocks meet
// at a bounded grid barrier between the reduction and the normalisation, when GEEPS_BN_COOP=1 (measured slower than the
// two launches, so it is off by default).
int geeps_bn_forward_fused(const void* x, void* y, const float* gamma, const float* beta, float* sums,
                           float* mean_rstd, float* running_mean, float* running_var, float* zero_after, int* barrier,
                           long long P, int C, long long ldx, long long ldy, float eps, float momentum, int relu,
                           void* stream);
int geeps_bn_backward_fused(const void* x, const void* dy, const void* y, void* dx, float* mean_rstd,
                            const float* gamma, float* sums, float* dgamma, float* dbeta, float* zero_after,
                            int* barrier, long long P, int C, long long ldx, long long lddy, long long lddx, int relu,
                            float grad_scale, void* stream);
// out[c] (+)= scale * sum_p x[p][c]
// dx = y > 0 ? dy : 0 and colsum[c] = sum over the P pixels of dx (C % 8 == 0, C <= 8192), one pass
int geeps_relu_backward_colsum(const void* dy, const void* y, void* dx, float* colsum, long long P, int C,
                               long long lddy, long long ldy, long long lddx, void* stream);
int geeps_colsum(const void* x, float* out, long long P, int C, long long ldx, float scale, int zero_first,
                 void* stream);
int geeps_relu_backward(const void* dy, const void* y, void* dx, long long n, void* stream);
int geeps_relu_backward_2d(const void* dy, const void* y, void* dx, long long P, int C, long long lddy, long long ldy,
                           long long lddx, void* stream);
// dst[P][C] (bf16) = src[P][C] (fp32), optionally through ReLU; row pitches in elements
int geeps_f32_to_bf16_2d(const float* src, void* dst, long long P, int C, long long lds, long long ldd, int relu,
                         void* stream);
int geeps_add_bf16_2d(void* dst, const void* src, long long P, int C, long long ldd, long long lds, void* stream);
int geeps_dropout(const void* x, void* y, long long n, float p, unsigned long long seed, void* stream);
// the same with the seed taken as seed + *step_ref when the kernel runs (a device-resident step counter: the launch
// arguments stay the same from step to step, so the launch can sit in a replayed CUDA graph)
int geeps_dropout_ref(const void* x, void* y, long long n, float p, unsigned long long seed, const int* step_ref,
                      void* stream);
// rscale: bf16 buffer [P][C] that receives 1 / scale for the backward pass
int geeps_lrn_forward(const void* x, void* y, void* rscale, long long P, int C, int size, float alpha, float beta,
                      float k, void* stream);
// relu_mask != 0: x is a ReLU output; its backward is folded in (dx = 0 where x <= 0)
int geeps_lrn_backward(const void* x, const void* y, const void* rscale, const void* dy, void* dx, long long P,
                       int C, int size, float alpha, float beta, int relu_mask, float* colsum, void* stream);
// colsum (or NULL): C floats that receive the per-channel sums of dx (C % 8 == 0, window 3 / 5 / 7 only)
int geeps_copy_f32(float* dst, const float* src, long long n, void* stream);
// LRN across channels fused with the max pooling after it (dense input: g->ldx == g->C; window 3 / 5 / 7).
// Forward keeps only the pooled tensor and the window codes; backward recomputes the normalisation from x and
// delivers dx (gradient w.r.t. the LRN input) with an optional ReLU mask (x <= 0 -> 0) and, in colsum (C floats
// or NULL), the per-channel sums of dx.
int geeps_lrn_maxpool_supported(const GeepsPoolGeom* g, int size);
int geeps_lrn_maxpool_forward(const void* x, void* p, void* argmax, const GeepsPoolGeom* g, int size, float alpha,
                              float beta, float k, void* stream);
int geeps_lrn_maxpool_backward(const void* x, const void* dp, const void* argmax, void* dx, const GeepsPoolGeom* g,
                               int size, float alpha, float beta, float k, int relu_mask, float* colsum, void* stream);
int geeps_maxpool_forward(const void* x, void* y, void* argmax, const GeepsPoolGeom* g, void* stream);
int geeps_maxpool_backward(const void* dy, const void* argmax, void* dx, const GeepsPoolGeom* g, int accumulate,
                           void* stream);
int geeps_avgpool_forward(const void* x, void* y, const GeepsPoolGeom* g, void* stream);
int geeps_avgpool_backward(const void* dy, void* dx, const GeepsPoolGeom* g, int accumulate, void* stream);
int geeps_softmax_ce(const float* logits, const long long* labels, float* loss_sum, float* per_sample,
                     void* dlogits, int B, int C, long long ldl, long long ldd, float loss_scale, float grad_scale,
                     int zero_loss, int* status, void* stream);

// ---- allocation-free BatchNorm forward (no counterpart in the reference, which has no layer kernels) ----
// Same result as geeps_bn_forward, but the 2*C floats of reduction scratch come from a fixed device
// array inside the library (GEEPS_BN_NOALLOC_MAX_CHANNELS channels, 32 KB per GPU, held until exit)
// instead of from the caller.  It is meant for callers that cannot allocate: code under the parameter
// server's fully planned GPU budget, and hosts without a device allocator that must keep cudaMalloc's
// device-wide synchronisation out of their step loop.  The call itself never calls cudaMalloc / cudaFree
// or any allocating library routine.
//  * C must be a multiple of 8 and <= GEEPS_BN_NOALLOC_MAX_CHANNELS; a larger C is rejected with
//    GEEPS_ERR_NOALLOC_TOO_LARGE (and a message on stderr) without launching anything.
//  * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
//    device current); make that first call before any stream capture begins.
//  * All calls share the one array, which keeps the previous call's contents; the part in use is cleared
//    on `stream` first.  Calls whose kernels may overlap on the GPU race on it: keep them on one stream
//    or order them with events.
#define GEEPS_BN_NOALLOC_MAX_CHANNELS 4096
#define GEEPS_ERR_NOALLOC_TOO_LARGE (-2)
int geeps_bn_noalloc_max_channels(void);
int geeps_bn_forward_noalloc(const void* x, void* y, const float* gamma, const float* beta, float* mean_rstd,
                             float* running_mean, float* running_var, long long P, int C, long long ldx,
                             long long ldy, float eps, float momentum, int relu, void* stream);

#ifdef __cplusplus
}
#endif
