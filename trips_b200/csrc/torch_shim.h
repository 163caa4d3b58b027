// libtorch host side of the rasterizer: the reference's operator interface on top of the C ABI (include/trips_b200.h).
//
// A TRIPS build includes this header instead of src/lib/rendering/PointRenderer.h / RenderModule.h and
// src/lib/models/MyAdam.h and links libtrips_b200_torch.so.  Names and argument order follow the reference:
//   NeuralRenderInfo, PointRendererCache, BlendPointCloud        PointRenderer.h:23-53, RenderInfo.cpp:14-40
//   PointRenderModule (forward(NeuralRenderInfo*))                RenderModule.h:10-27, RenderModule.cpp:44-110
//   MyAdamOptions, MyAdam (step, shrinkInternalState,
//     appendToInternalState), UpdateOptimLR                       MyAdam.h:29-118, MyAdam.cu:164-415
//   NeuralPointCloudCuda, NeuralPointTexture, PoseModule,
//     IntrinsicsModule (the registered tensor names = the
//     checkpoint format read by torch::load)                      NeuralPointCloudCuda.cpp:103-108, NeuralTexture.cpp:53-55,
//                                                                 NeuralStructure.cpp:34-35,142
// The reference reaches its tensors through NeuralScene; here NeuralRenderInfo holds the same tensors directly.
// Nothing is computed on the host: tensors are flattened to device pointers and handed to the C ABI on the current
// CUDA stream.
#pragma once
#include <torch/custom_class.h>
#include <torch/torch.h>

#include <memory>
#include <string>
#include <tuple>
#include <vector>

#include "trips_b200.h"

namespace trips_b200
{
using torch::Tensor;

// owns the C context, like PointRendererCache owns the reference's scratch tensors (PointRenderer.h:126-176)
struct PointRendererCache
{
    TripsContext* handle = nullptr;
    int device           = -1;
    Tensor dropout_points;  // [B,N], training with dropout > 0 only (PointRenderer.cu:518-523)
    ~PointRendererCache();
    void ensure(int dev);
};

struct NeuralRenderInfo : torch::CustomClassHolder
{
    // scene (NeuralScene: point_cloud_cuda, texture, poses, intrinsics)
    Tensor texture, background_color, t_position, poses_se3, tangent_poses, intrinsics, confidence_value_of_point, t_point_size, t_index;
    std::vector<TripsView> images;  // ReducedImageInfo, SceneData.h:40-61
    TripsRenderParams params{8, 16, 0, 0, 0.f, 0, 0.f, 0, 0, 10.f, 0, 1, 1, 0, 0, 0, 20.f};  // the reference's defaults (Settings.h)
    double dropout     = 0.0;
    int64_t num_layers = 8;
    bool train         = false;
    std::shared_ptr<PointRendererCache> cache = std::make_shared<PointRendererCache>();

    void set_scene(Tensor texture_, Tensor background_color_, Tensor t_position_, Tensor poses_se3_, c10::optional<Tensor> tangent_poses_,
                   Tensor intrinsics_, Tensor confidence_, Tensor t_point_size_, c10::optional<Tensor> t_index_);
    void add_image(int64_t w, int64_t h, int64_t image_index, int64_t camera_index, int64_t camera_model_type,
                   std::vector<double> crop_transform, std::vector<double> crop_rotation);
    void clear_images();
    // RenderParams fields of the live path (Settings.h:19-108) + NeuralRenderInfo::num_layers / train
    void set_params(int64_t num_layers_, int64_t k_keep, bool train_, bool drop_out_points_by_radius, double drop_out_radius_threshold,
                    bool viewer_only, double stability_cutoff_value, bool bg_uses_Tn, double dropout_);
    // texture preparation fused into the rasterizer (NeuralTexture.h:40-57): the tensors given to set_scene are the raw ones
    void set_texture_preparation(bool confidence_is_raw, double confidence_scale, bool texture_abs);
    // the flags that select the reference's second forward pipeline (RenderParams, Settings.h; PointRenderer.cu:730-731)
    void set_pipeline_flags(bool use_layer_point_size, bool render_points_in_all_lower_resolutions, bool combine_lists,
                            bool saturated_alpha_accumulation);
    // lens distortion: apply the 8 coefficients of the intrinsics rows and the cut-off radius (RenderParams::dist_cutoff)
    void set_distortion(bool distortion, double dist_cutoff);
    int64_t last_status();
};

// BlendPointCloud (RenderInfo.cpp:27-40): one tensor [B,C,H_l,W_l] per layer, differentiable with respect to texture,
// background, positions, pose tangents, intrinsics, confidences and point sizes.
std::vector<Tensor> BlendPointCloud(const c10::intrusive_ptr<NeuralRenderInfo>& info);

// PointRenderModuleImpl (RenderModule.h:10-27): owns one cache that every forward call reuses; returns (images, masks)
// with masks empty (output_background_mask is not implemented).
struct PointRenderModuleImpl : torch::nn::Module
{
    explicit PointRenderModuleImpl(int num_layers_);
    std::pair<std::vector<Tensor>, std::vector<Tensor>> forward(const c10::intrusive_ptr<NeuralRenderInfo>& nri);
    int num_layers;
    std::shared_ptr<PointRendererCache> cache;
};
TORCH_MODULE(PointRenderModule);

// ---- MyAdam (MyAdam.h:29-85) ----
struct MyAdamOptions : public torch::optim::OptimizerCloneableOptions<MyAdamOptions>
{
    MyAdamOptions(double lr = 1e-3) { set_lr(lr); }
    TORCH_ARG(double, lr) = 1e-3;
    typedef std::tuple<double, double> betas_t;
    TORCH_ARG(betas_t, betas)                    = std::make_tuple(0.9, 0.999);
    TORCH_ARG(double, eps)                       = 1e-8;
    TORCH_ARG(double, relative_weight_decay)     = 0;
    TORCH_ARG(double, absolute_weight_decay)     = 0;
    TORCH_ARG(double, weight_clipping_magnitude) = 0;
    TORCH_ARG(bool, adabound)                    = false;

   public:
    ~MyAdamOptions() override = default;
    double get_lr() const override { return lr(); }
    void set_lr(const double lr) override { this->lr(lr); }
};

struct MyAdamParamState : public torch::optim::OptimizerCloneableParamState<MyAdamParamState>
{
    TORCH_ARG(Tensor, param_steps);  // int32 per element (the reference keeps int64)
    TORCH_ARG(Tensor, first_moments);
    TORCH_ARG(Tensor, second_moments);
    TORCH_ARG(int64_t, current_step) = 0;

   public:
    ~MyAdamParamState() override = default;
};

class MyAdam : public torch::optim::Optimizer
{
   public:
    explicit MyAdam(std::vector<torch::optim::OptimizerParamGroup> param_groups, MyAdamOptions defaults = {});
    explicit MyAdam(std::vector<Tensor> params, MyAdamOptions defaults = {});
    ~MyAdam() override;
    // One kernel launch over all parameters of all groups (the reference launches adam_step per tensor, MyAdam.cu:226-280).
    Tensor step(LossClosure closure = nullptr) override;
    void save(torch::serialize::OutputArchive& archive) const override;  // not supported, as in the reference (MyAdam.cu:417-425)
    void load(torch::serialize::InputArchive& archive) override;
    // keep the listed entries along the last dimension of every state tensor of the group (MyAdam.cu:346-373)
    void shrinkInternalState(int param_group_index, Tensor indices_to_keep);
    // zero-extend every state tensor of the group along its last dimension (MyAdam.cu:376-415)
    void appendToInternalState(int param_group_index, int new_size);
    // state of one parameter, or nullptr before its first step
    MyAdamParamState* state_of(const Tensor& p);

   private:
    TripsContext* ctx_ = nullptr;
    int device_        = -1;
};

void UpdateOptimLR(torch::optim::Optimizer* optimizer, double factor);  // MyAdam.h:91-118

// ---- parameter modules: the registered names are the checkpoint format (torch::save / torch::load of the module) ----
struct NeuralPointCloudCudaImpl : torch::nn::Module
{
    NeuralPointCloudCudaImpl(Tensor position /*[N,4]*/, Tensor point_size /*[N,1]*/, Tensor index /*[N,1] int32*/, Tensor original_color /*[N,4]*/);
    Tensor t_position, t_point_size, t_index, t_original_color;
};
TORCH_MODULE(NeuralPointCloudCuda);

struct NeuralPointTextureImpl : torch::nn::Module
{
    NeuralPointTextureImpl(int num_channels, int num_points);
    Tensor texture_raw, background_color_raw, confidence_raw;  // registered as texture, background_color, confidence_value_of_point
};
TORCH_MODULE(NeuralPointTexture);

struct PoseModuleImpl : torch::nn::Module
{
    explicit PoseModuleImpl(int num_images);
    Tensor tangent_poses, poses_se3;
};
TORCH_MODULE(PoseModule);

struct IntrinsicsModuleImpl : torch::nn::Module
{
    explicit IntrinsicsModuleImpl(int num_cameras);
    Tensor intrinsics;
};
TORCH_MODULE(IntrinsicsModule);
}  // namespace trips_b200
