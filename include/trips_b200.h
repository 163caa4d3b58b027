/* trips_b200 -- C ABI of the B200 (sm_100a) point-splatting rasterizer, its backward pass and the fused Adam.
 *
 * This is the boundary a TRIPS build binds instead of its own CUDA kernels.  Every entry point replaces one
 * piece of the reference (paths relative to the lfranke/TRIPS source tree); all data pointers are DEVICE
 * pointers owned by the caller unless stated otherwise, layouts are the reference's own tensor layouts, and
 * work is enqueued on the given stream.  Functions return TRIPS_OK (0) or a negative TripsStatus; no entry
 * point aborts the process or traps the device (the reference uses SAIGA_ASSERT / CUDA_KERNEL_ASSERT).
 */
#ifndef TRIPS_B200_H
#define TRIPS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TRIPS_MAX_LAYERS 8  /* src/lib/rendering/RenderConstants.h:38 */
#define TRIPS_MAX_KEEP 16   /* src/lib/rendering/PointRenderer.h:178 (max_pixels_per_list) */
#define TRIPS_MAX_CHANNELS 16

typedef enum
{
    TRIPS_OK                  = 0,
    TRIPS_ERR_INVALID_ARG     = -1,
    TRIPS_ERR_CUDA            = -2,
    TRIPS_ERR_OUT_OF_MEMORY   = -3,
    TRIPS_ERR_UNSUPPORTED     = -4, /* camera model / flag outside the implemented live path */
    TRIPS_ERR_NO_FORWARD      = -5, /* backward without a matching training forward */
    TRIPS_ERR_TOO_LARGE       = -6  /* size beyond a stated maximum */
} TripsStatus;

/* Bits of the device status word (trips_last_status): conditions the reference would assert on. */
#define TRIPS_DEV_BAD_TEXTURE_INDEX 1u /* RenderBackward.cu:217-218 */
#define TRIPS_DEV_NONZERO_DISTORTION 2u /* non-zero distortion coefficients while TripsRenderParams.distortion = 0: they were ignored */
#define TRIPS_DEV_FRAGMENT_OVERFLOW 4u /* a view's fragments did not fit the list buffer (sized from the previous call): the view was rendered as background; the next call grows the buffer */
#define TRIPS_DEV_BAD_FRAGMENT 8u /* a fragment referred to a point outside the view's visible set (internal error) */
#define TRIPS_DEV_BAD_POINT_INDEX 16u /* trips_resize_points: a removal index is out of range or listed twice */
#define TRIPS_DEV_ENTRY_OVERFLOW 32u /* a view's visible points did not fit the entry arrays (sized from the previous call): same handling as TRIPS_DEV_FRAGMENT_OVERFLOW */

typedef struct TripsContext TripsContext;

/* The scene as the reference's modules hold it.
 * position, point_size, index: NeuralPointCloudCuda (src/lib/rendering/NeuralPointCloudCuda.h:78-96);
 * texture, confidence, background: NeuralPointTexture after PrepareTexture / PrepareConfidence
 * (src/lib/models/NeuralTexture.h:40-57); poses: PoseModule::poses_se3, intrinsics: IntrinsicsModule::intrinsics
 * (src/lib/data/NeuralStructure.cpp:20-33,104-117), both read through DeviceRenderParams (RenderConstants.h:85-100). */
typedef struct
{
    int n_points;             /* N */
    int n_tex;                /* columns of texture / confidence */
    int channels;             /* C: 3, 4, 6, 8 or 16 */
    const float* position;    /* [N,4] xyz + drop-out radius */
    const float* point_size;  /* [N] softplus-parametrised world-space size */
    const int32_t* index;     /* [N] point -> texture column; NULL = identity */
    const float* texture;     /* [C,n_tex] */
    const float* confidence;  /* [n_tex] activated confidence */
    const float* background;  /* [C] */
    const float* dropout;     /* [B,N] 1 = point dropped in that view (training only); NULL = none */
    const double* poses;      /* [n_images,8] world->view: quaternion x,y,z,w, translation x,y,z, pad */
    int n_images;
    const float* intrinsics;  /* [n_cameras,13] fx fy cx cy s + 8 distortion coefficients k1 k2 k3 k4 k5 k6 p1 p2 */
    int n_cameras;
} TripsScene;

/* One view = ReducedImageInfo (src/lib/data/SceneData.h:40-61).  crop_rotation is row-major. */
typedef struct
{
    int w, h;
    int image_index;
    int camera_index;
    int camera_model_type; /* 0 = PINHOLE_DISTORTION, the only model implemented */
    float crop_transform[5]; /* fx fy cx cy s */
    float crop_rotation[4];
} TripsView;

/* The RenderParams fields the live path reads (src/lib/data/Settings.h:19-108, RenderConstants.h:115-140). */
typedef struct
{
    int num_layers;                  /* 1..8 */
    int k_keep;                      /* fragments kept per pixel, 1..16 (reference: 16) */
    int train;                       /* 1: keep backward records, honour dropout */
    int drop_out_points_by_radius;
    float drop_out_radius_threshold;
    int viewer_only;                 /* 1: discard points with confidence < stability_cutoff_value */
    float stability_cutoff_value;
    int bg_uses_Tn;                  /* 0 = reference behaviour for the background weight */
    /* Texture preparation fused into the pass that gathers the per-point data (NeuralTexture.h:40-57: the reference
     * runs sigmoid((10 + narrowing) * raw) over [1,N] and abs over [C,N] as separate torch ops every step, and their
     * backward).  When set, TripsScene.confidence / .texture hold the RAW parameters and the gradients returned by
     * trips_backward are those of the raw parameters. */
    int confidence_is_raw;           /* 1: confidence = sigmoid(confidence_scale * raw) */
    float confidence_scale;          /* 10 + narrowing factor */
    int texture_abs;                 /* 1: descriptor = |raw| */
    /* The flags whose non-default values select the reference's second forward pipeline (PointRenderer.cu:730-731:
     * CountTiled, CollectTiled2[Pointsize], FastSortAndBlendWPrep2WarpSharedWork, RenderForward.cu:1401-3674).  The
     * reference's defaults are 1, 1, 0, 0 (Settings.h); a zero-initialised struct does NOT hold the defaults. */
    int use_layer_point_size;                   /* 0: a point is written to every layer, alpha carries no layer factor */
    int render_points_in_all_lower_resolutions; /* 0: only the two layers around log2(size) are written (RenderForward.cu:2291-2393) */
    int combine_lists;                          /* 1: a pixel also draws from the lists of the pixels above it on the coarser layers (RenderForward.cu:3232-3242) */
    int saturated_alpha_accumulation;           /* forward: second pipeline only (RenderForward.cu:3524-3548; compiled out of the
                                                   first, :908-935); backward: always (RenderBackward.cu:227-259) */
    /* Lens distortion of ProjectPointPinholeWoNormal / ProjectPointPinholeBackward (PointRendererHelper.h:232-253,
     * 434-494): the 8-coefficient rational model with tangential terms of saiga's distortNormalizedPoint,
     * x' = x (1 + k1 r2 + k2 r4 + k3 r6) / (1 + k4 r2 + k5 r4 + k6 r6) + 2 p1 x y + p2 (r2 + 2 x^2), y' alike; points with
     * r2 > dist_cutoff^2 are culled.  1: applied, and the intrinsics gradient carries all 13 entries.  0: a plain
     * pinhole (the coefficients must be zero, TRIPS_DEV_NONZERO_DISTORTION otherwise; no cut-off radius). */
    int distortion;
    float dist_cutoff;                          /* RenderParams::dist_cutoff (Settings.h:61: 20) */
} TripsRenderParams;

/* Gradient outputs of BlendPointCloudBackward (src/lib/rendering/PointRenderer.cu:1423-1426).
 * Any pointer may be NULL (that gradient is not produced).  Buffers are overwritten, not accumulated. */
typedef struct
{
    float* texture;      /* [C,n_tex] */
    float* background;   /* [C] */
    float* points;       /* [N,4], w = 0 */
    double* pose_tangent; /* [n_images,6] */
    float* intrinsics;   /* [n_cameras,13]; the 8 distortion coefficients receive gradients when TripsRenderParams.distortion is set */
    float* confidence;   /* [n_tex] */
    float* point_size;   /* [N] ("g_layer") */
} TripsGrads;

/* Counters of the last forward call, summed over its views. */
typedef struct
{
    int64_t visible_points; /* V */
    int64_t fragments;      /* F */
    int64_t kept_fragments; /* Kf = sum over pixels of min(list length, k_keep) */
    int64_t pixels;         /* B * P */
    int64_t max_list_length;
    int64_t culled_point_blocks; /* (view, block of 8192 consecutive points) pairs skipped by the bounding-box frustum test */
} TripsStats;

/* Context = PointRendererCache (src/lib/rendering/PointRenderer.h:120-232): owns all scratch memory and the
 * records saved for backward.  One context per device and per concurrent stream. */
int trips_context_create(TripsContext** out, int device);
void trips_context_destroy(TripsContext* ctx);
const char* trips_status_string(int status);
const char* trips_last_error(const TripsContext* ctx);

/* Replaces BlendPointCloudForward / PointRendererCache::RenderFast16
 * (src/lib/rendering/PointRenderer.cu:676-1191, RenderForward.cu:1065-1394).
 * out_layers: HOST array of num_layers device pointers; layer l is [B,C,H_l,W_l] float32 contiguous with
 * ceil-halved sizes (PointRenderer.cu:385-389).  All views must share (w, h). */
int trips_forward(TripsContext* ctx, const TripsScene* scene, const TripsView* views, int n_views,
                  const TripsRenderParams* params, float* const* out_layers, void* stream);

/* Replaces BlendPointCloudBackward / BlendBackwardsBilinearFast
 * (src/lib/rendering/PointRenderer.cu:1232-1427, RenderBackward.cu:90-691).  Uses the records of the last
 * trips_forward on this context.  grad_layers: HOST array of num_layers device pointers, same shapes as out_layers. */
int trips_backward(TripsContext* ctx, const TripsScene* scene, const float* const* grad_layers, const TripsGrads* grads,
                   void* stream);

/* Blocks until the stream is idle and returns the OR of device status bits raised since the last call. */
uint32_t trips_last_status(TripsContext* ctx, void* stream);
int trips_get_stats(TripsContext* ctx, TripsStats* out, void* stream);

/* One parameter tensor of MyAdam (src/lib/models/MyAdam.cu:164-345): weights, gradient and optimizer state. */
typedef struct
{
    float* weights;
    const float* gradients;
    float* first_moments;
    float* second_moments;
    int32_t* steps; /* per-element step counter (the reference keeps int64) */
    int64_t n;
    float lr;
    float beta1, beta2, eps;
    float relative_weight_decay, absolute_weight_decay, weight_clipping_magnitude;
    float lower_lr_bound, upper_lr_bound; /* AdaBound bounds; 0 and FLT_MAX when off */
} TripsAdamTensor;

/* Replaces MyAdam::step's per-tensor adam_step launches (src/lib/models/MyAdam.cu:41-88,226-280) with one
 * launch over all tensors.  `tensors` is a HOST array. */
int trips_adam_step(TripsContext* ctx, const TripsAdamTensor* tensors, int n_tensors, void* stream);

/* View-parallel training over several GPUs of one node (no counterpart in the reference, which is single-GPU:
 * its views meet only in the gradient buffers filled by the sequential view loop, PointRenderer.cu:1339-1344).
 * All point parameters live in ONE flat fp32 buffer per rank and all their gradients in another, both mapped into
 * every rank's address space (peer memory).  A segment describes one parameter tensor inside the flat space. */
#define TRIPS_MAX_RANKS 16
#define TRIPS_MAX_SEGMENTS 8
typedef struct
{
    int64_t offset; /* first flat element of the tensor; segments are sorted by offset, the first one starts at 0 */
    float lr;
    float beta1, beta2, eps;
    float relative_weight_decay, absolute_weight_decay, weight_clipping_magnitude;
    float lower_lr_bound, upper_lr_bound;
} TripsAdamSegment;

/* Sums the gradients of all ranks for the flat elements [lo, hi) owned by this rank (peer loads, rank order),
 * applies the MyAdam update (src/lib/models/MyAdam.cu:41-88) with this rank's slice of the optimizer state
 * (first_moments / second_moments / steps hold hi - lo elements) and stores the new weights into the parameter
 * buffer of every rank (peer stores).  grad_ptrs / param_ptrs: HOST arrays of `world` device pointers to the flat
 * buffers of ranks 0..world-1 as mapped on THIS device.  The caller must order the call after the backward pass of
 * every rank and the next forward pass of every rank after it (a barrier before and after); the kernel itself
 * never waits on a peer.  lo and hi need no alignment. */
int trips_fused_reduce_adam(TripsContext* ctx, const float* const* grad_ptrs, float* const* param_ptrs, int world, int rank,
                            const TripsAdamSegment* segments, int n_segments, int64_t lo, int64_t hi, float* first_moments,
                            float* second_moments, int32_t* steps, void* stream);

/* The same step through NVSwitch multicast addresses (multimem.ld_reduce / multimem.st): grad_multicast and
 * param_multicast are the multicast mappings of the flat gradient buffers and of the flat parameter replicas of all
 * ranks (e.g. the multicast_ptr of a symmetric-memory allocation), param_local is this rank's replica.  Half the
 * NVLink bytes of trips_fused_reduce_adam.  The switch sums in an order of its own: weights equal
 * trips_fused_reduce_adam's bit for bit with two ranks only; replicas are identical with any number of ranks.
 * lo and hi must be multiples of 4 elements.  Ordering as for trips_fused_reduce_adam: the kernel waits on nothing. */
int trips_fused_reduce_adam_multicast(TripsContext* ctx, const float* grad_multicast, float* param_multicast, const float* param_local,
                                      const TripsAdamSegment* segments, int n_segments, int64_t lo, int64_t hi, float* first_moments,
                                      float* second_moments, int32_t* steps, void* stream);

/* One per-point tensor of the scene or of the optimizer state for trips_resize_points. */
typedef struct
{
    const void* src;     /* old tensor */
    void* dst;           /* new tensor, n_new points, allocated by the caller; must not overlap src */
    int rows;            /* values per point: 4 for t_position, C for the texture, 1 for sizes / confidences / step counters */
    int elem_bytes;      /* 4 or 8 */
    int point_major;     /* 1: [N, rows] (t_position, t_point_size); 0: [rows, N] (texture, confidence and their Adam state) */
    uint32_t fill_bits;  /* bit pattern of the value for appended points (0.5f for the texture, 0 for optimizer state) */
} TripsPointTensor;
#define TRIPS_MAX_POINT_TENSORS 32

/* Replaces the removal / growth of points over all per-point tensors and the optimizer state:
 * NeuralScene::RemovePoints (src/lib/data/NeuralScene.cpp:1375-1431: host sort, CPU mesh rebuild, one index_select
 * per tensor), NeuralPointTextureImpl::RemoveAndFlatten / ResizeAndFill (src/lib/models/NeuralTexture.cpp:153-208),
 * MyAdam::shrinkInternalState / appendToInternalState (src/lib/models/MyAdam.cu:346-415).
 * indices_to_remove: device array of n_remove distinct point indices in any order (the reference sorts them on the
 * host), may be NULL when n_remove is 0.  Every dst receives the kept points in their old order followed by
 * n_new - (n_points - n_remove) appended points holding the tensor's fill value; n_new must not be smaller than the
 * number of kept points.  One scan and one gather launch cover all tensors; nothing is copied to the host.  An index
 * out of range or listed twice raises TRIPS_DEV_BAD_POINT_INDEX in trips_last_status. */
int trips_resize_points(TripsContext* ctx, const int64_t* indices_to_remove, int64_t n_remove, int64_t n_points, int64_t n_new,
                        const TripsPointTensor* tensors, int n_tensors, void* stream);

/* No counterpart in the reference.  Same update as trips_adam_step for callers that cannot allocate device
 * memory at the time of the step: code running while the application's own pool owns all free memory, or hosts that
 * forbid cudaMalloc after start-up.  The table describing the tensors, which trips_adam_step keeps in cudaMalloc'ed
 * context scratch, lives here in a fixed array inside the library's device image, so the call performs no
 * cudaMalloc / cudaFree and needs no TripsContext.
 * Limits and rules: at most TRIPS_ADAM_STATIC_MAX_TENSORS tensors per call (more returns TRIPS_ERR_TOO_LARGE); the
 * array costs about 6 KB on every GPU that loads the library, until the process exits; the first call on a device
 * looks up the array's device address (with that device current) and should be made before any stream capture;
 * the table is uploaded from the call's own stack frame, so a stream that is being captured is refused with
 * TRIPS_ERR_UNSUPPORTED and nothing is enqueued; all calls on a device share the one array, which is rewritten by
 * each call, so two calls that may overlap on the GPU (different streams without ordering) race on it and must be
 * serialised by the caller. */
#define TRIPS_ADAM_STATIC_MAX_TENSORS 64
int trips_adam_step_static(const TripsAdamTensor* tensors, int n_tensors, void* stream);

/* Stage timers: CUDA-event pairs around every kernel stage, the counterpart of the reference's
 * SAIGA_OPTIONAL_TIME_MEASURE scopes (src/lib/rendering/RenderForward.cu:1090,1166,1238,1271,
 * PointRenderer.cu:1338) carried in NeuralRenderInfo::timer_system.  Off by default. */
enum
{
    TRIPS_STAGE_SETUP = 0,
    TRIPS_STAGE_BIN_POINTS,
    TRIPS_STAGE_COUNT,
    TRIPS_STAGE_SCAN,
    TRIPS_STAGE_COLLECT,
    TRIPS_STAGE_SORT_BLEND,
    TRIPS_STAGE_BACKWARD,
    TRIPS_STAGE_UNPACK,
    TRIPS_STAGE_ADAM,
    TRIPS_STAGE_LOSS,
    TRIPS_STAGE_FUSED_ADAM,
    TRIPS_STAGE_RESIZE,
    TRIPS_NUM_STAGES
};
int trips_enable_stage_timers(TripsContext* ctx, int enable);
/* Waits for the recorded events.  ms, timed_calls, kernel_launches: HOST arrays of TRIPS_NUM_STAGES entries (any
 * may be NULL): accumulated milliseconds, number of timed spans and number of kernels launched per stage since
 * the last reset (launches are counted whether or not the timers are on). */
int trips_get_stage_times(TripsContext* ctx, double* ms, int64_t* timed_calls, int64_t* kernel_launches, int reset);
const char* trips_stage_name(int stage);

/* Benchmark helper with no counterpart on the reference's renderer path (its losses live in
 * src/lib/models/Pipeline.cpp:703): for every pyramid layer grad = sign(out - target) / total_numel and
 * *loss_out (device double) = mean |out - target| over all layers.  The three pointer arrays and layer_numel
 * are HOST arrays of num_layers entries. */
int trips_l1_loss_backward(TripsContext* ctx, const float* const* out_layers, const float* const* target_layers,
                           float* const* grad_layers, const int64_t* layer_numel, int num_layers, double* loss_out,
                           void* stream);

/* ---- inspection of the intermediates of the last forward call (used by the parity tests) ---- */
/* Per-point results of view `view`: depth [N] (-1 = culled), nlayers [N] int32, record [N,4] (u, v, size_px, texture index bits).
 * HOST output pointers, any may be NULL.  RenderForward.cu:311-363. */
int trips_debug_points(TripsContext* ctx, int view, float* depth, int32_t* nlayers, float* record, void* stream);
/* Per-pixel list lengths [P] int32, start offsets [P] int64 (relative to the view's first fragment) and the
 * view's fragments (64-bit keys: depth bits << 32 | point id) in list order.  HOST pointers; pass frags = NULL
 * and read *n_frags first to size the buffer.  RenderForward.cu:387-413. */
int trips_debug_lists(TripsContext* ctx, int view, int32_t* counts, int64_t* offsets, uint64_t* frags, int64_t* n_frags,
                      void* stream);
/* Backward records of view `view`: nrec [P] int32, point ids [P,16] int32 (-1 = absent), alphas [P,16] (-1 = absent).
 * RenderForward.cu:957-979. */
int trips_debug_records(TripsContext* ctx, int view, int32_t* nrec, int32_t* rec_pid, float* rec_alpha, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TRIPS_B200_H */
