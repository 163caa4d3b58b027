/* CPU oracle for the TRIPS trilinear point-splatting hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain C++17 / OpenMP restatement of the reference's CUDA kernels (lfranke/TRIPS,
 * src/lib/rendering/RenderForward.cu, RenderBackward.cu, PointBlending.h, PointRendererHelper.h and
 * src/lib/models/MyAdam.cu).  It exists to check the CUDA library and to be timed as the CPU baseline;
 * nothing in the shipped package may call it.
 *
 * PARITY UNPINNED: the reference has no tests, fixtures or golden vectors for this path and cannot be
 * compiled without its un-vendored `saiga` submodule, so this restatement is pinned only by hand-derived
 * known-answer cases and finite-difference checks, not by reference outputs.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct
{
    int n_points;            /* N */
    int n_tex;               /* columns of texture / confidence */
    int channels;            /* C */
    const float* position;   /* [N,4] xyz + drop-out radius */
    const float* point_size; /* [N] raw, softplus-parametrised */
    const int32_t* index;    /* [N] point -> texture column, or NULL for identity */
    const float* texture;    /* [C, n_tex] */
    const float* confidence; /* [n_tex], already sigmoid-activated */
    const float* background; /* [C] */
    const float* dropout;    /* [N] per-view mask (1 = dropped) or NULL */
} OrScene;

typedef struct
{
    int w, h;
    double pose[8];         /* world->view: quaternion x,y,z,w then translation x,y,z, one pad */
    float intrinsics[13];   /* fx fy cx cy s + 8 distortion coefficients k1..k6 p1 p2 (applied when OrParams.distortion) */
    float crop_transform[5]; /* fx fy cx cy s */
    float crop_rotation[4]; /* row-major 2x2 */
} OrView;

typedef struct
{
    int num_layers;
    int k_keep; /* fragments kept per pixel, <= 16 */
    int train;
    int drop_out_points_by_radius;
    float drop_out_radius_threshold;
    int viewer_only;
    float stability_cutoff_value;
    int bg_uses_Tn; /* 0 = reference behaviour (weight before the last kept fragment) */
    /* The flags that select the reference's second forward pipeline (PointRenderer.cu:730-731: CountTiled,
     * CollectTiled2[Pointsize], FastSortAndBlendWPrep2WarpSharedWork) when they differ from 1, 1, 0. */
    int use_layer_point_size;                   /* 0: every layer is written, no layer factor */
    int render_points_in_all_lower_resolutions; /* 0: only the two layers around log2(size) are written */
    int combine_lists;                          /* 1: a pixel also draws from the lists of the coarser layers above it */
    int saturated_alpha_accumulation;           /* forward: second pipeline only (RenderForward.cu:3524-3548; compiled out
                                                   of the first, :908-935); backward: always (RenderBackward.cu:227-259) */
    /* Lens distortion of ProjectPointPinholeWoNormal (PointRendererHelper.h:232-253).  distortNormalizedPoint lives in
     * the saiga library (External/saiga, not part of the reference tree): restated here as the 8-coefficient rational
     * model with tangential terms that saiga's Distortion struct documents (OpenCV's k1 k2 p1 p2 k3 k4 k5 k6 model),
     * coefficient order k1 k2 k3 k4 k5 k6 p1 p2, points with x^2 + y^2 > dist_cutoff^2 culled (the reference tests
     * for the 100000 the routine returns there, PointRendererHelper.h:246-249).  UNPINNED like the rest. */
    int distortion;    /* 0: coefficients must be zero and dist_cutoff is not applied */
    float dist_cutoff; /* RenderParams::dist_cutoff, Settings.h:61 (20) */
} OrParams;

typedef struct OrFrame OrFrame; /* all intermediates of one rendered view */

int or_max_threads(void);
void or_sigmoid(const float* raw, float scale, float* out, long long n); /* NeuralTexture.h:40-43 */
void or_set_threads(int n); /* OpenMP team size of the following calls (launchers may export OMP_NUM_THREADS=1) */

OrFrame* or_forward(const OrScene* scene, const OrView* view, const OrParams* params);
void or_frame_free(OrFrame* f);

int64_t or_num_pixels(const OrFrame* f);    /* P */
int64_t or_num_fragments(const OrFrame* f); /* F */
int64_t or_num_kept(const OrFrame* f);      /* Kf = sum min(len, K) */
int64_t or_num_visible(const OrFrame* f);   /* V */
void or_layer_size(const OrFrame* f, int layer, int* w, int* h, int64_t* base);

/* copy-outs; every pointer may be NULL */
void or_get_points(const OrFrame* f, float* depth /*[N]*/, int32_t* nlayers /*[N]*/, float* rec /*[N,4] u v ps texidx-bits*/);
void or_get_first_layer(const OrFrame* f, int32_t* first /*[N] first layer each point is written to*/);
void or_get_lists(const OrFrame* f, int32_t* counts /*[P]*/, int64_t* offsets /*[P]*/, uint64_t* frags /*[F]*/);
void or_get_pyramid(const OrFrame* f, float* out /*[sum_l C*H_l*W_l], layer-major, channel-planar*/);
void or_get_records(const OrFrame* f, int32_t* nrec /*[P]*/, int32_t* rec_pid /*[P,16]*/, float* rec_alpha /*[P,16]*/);

/* Backward of one view.  grad_pyramid has the layout of or_get_pyramid.  Outputs are ACCUMULATED in double. */
void or_backward(const OrFrame* f, const OrScene* scene, const OrView* view, const OrParams* params,
                 const float* grad_pyramid, double* g_texture /*[C,n_tex]*/, double* g_confidence /*[n_tex]*/,
                 double* g_position /*[N,4], w untouched*/, double* g_point_size /*[N]*/,
                 double* g_background /*[C]*/, double* g_pose /*[6] or NULL*/,
                 double* g_intrinsics /*[13] or NULL: fx fy cx cy s, then the 8 distortion coefficients*/);

/* Reference Adam (MyAdam.cu:41-88) over n elements; steps is int64 per element. */
void or_adam(int64_t n, float* w, const float* g, float* m, float* v, int64_t* steps, float lr, float beta1,
             float beta2, float eps, float rel_decay, float abs_decay, float clip, float lower_lr, float upper_lr);

/* primitives exposed for known-answer tests */
float or_layer_factor(float ps, int layer, int num_layers, float* grad);
float or_softplus(float x);
float or_expf(float x);
float or_logf(float x);
void or_project(const OrView* view, const float* p3, float* u, float* v, float* z);

/* diagnostics for the parity report: out[6] = visible points, visible with ps > 1, points whose exact-bits ceil(log2 ps)
 * differs from ceil(log2f(ps)) of the host libm (RenderForward.cu:345), the same for floor, points whose layer count
 * would change with a libm softplus, points whose softplus differs in any bit from the libm one */
void or_layer_divergence(const OrFrame* f, const OrScene* scene, const OrView* view, const OrParams* params, int64_t* out);
/* largest error (ulp of the float result) of the reproducible exp / log against double-precision libm, every stride-th float */
void or_math_sweep(uint32_t stride, double* max_ulp_exp, double* max_ulp_log);

#ifdef __cplusplus
}
#endif
