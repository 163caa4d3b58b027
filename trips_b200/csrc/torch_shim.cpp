// libtorch host side of the rasterizer (see torch_shim.h): NeuralRenderInfo / PointRender / BlendPointCloud /
// PointRenderModule / MyAdam and the parameter modules, all on top of the C ABI.  Also registered for Python as
// torch.classes.trips_b200.{NeuralRenderInfo, PointRenderModule, MyAdam} and torch.ops.trips_b200.{blend_point_cloud,
// adam_step}, which is how tests/ drive this file.
#include "torch_shim.h"

#include <c10/cuda/CUDAStream.h>

#include <mutex>
#include <stdexcept>

namespace trips_b200
{
static void check(int st, TripsContext* ctx, const char* what)
{
    if (st != TRIPS_OK) throw std::runtime_error(std::string(what) + ": " + trips_status_string(st) + " (" + trips_last_error(ctx) + ")");
}

// ------------------------------------------------------------------------------------------------------------
// PointRendererCache, NeuralRenderInfo
// ------------------------------------------------------------------------------------------------------------
PointRendererCache::~PointRendererCache()
{
    if (handle) trips_context_destroy(handle);
}

void PointRendererCache::ensure(int dev)
{
    if (handle && dev == device) return;
    if (handle) trips_context_destroy(handle);
    handle       = nullptr;
    const int st = trips_context_create(&handle, dev);
    if (st != TRIPS_OK) throw std::runtime_error(std::string("trips_context_create: ") + trips_status_string(st));
    device = dev;
}

void NeuralRenderInfo::set_scene(Tensor texture_, Tensor background_color_, Tensor t_position_, Tensor poses_se3_,
                                 c10::optional<Tensor> tangent_poses_, Tensor intrinsics_, Tensor confidence_, Tensor t_point_size_,
                                 c10::optional<Tensor> t_index_)
{
    texture = texture_, background_color = background_color_, t_position = t_position_, poses_se3 = poses_se3_;
    tangent_poses = tangent_poses_.has_value() ? *tangent_poses_ : Tensor();
    intrinsics = intrinsics_, confidence_value_of_point = confidence_, t_point_size = t_point_size_;
    t_index = t_index_.has_value() ? *t_index_ : Tensor();
}

void NeuralRenderInfo::add_image(int64_t w, int64_t h, int64_t image_index, int64_t camera_index, int64_t camera_model_type,
                                 std::vector<double> crop_transform, std::vector<double> crop_rotation)
{
    TORCH_CHECK(crop_transform.size() == 5 && crop_rotation.size() == 4, "crop_transform has 5, crop_rotation 4 values");
    TripsView v{};
    v.w = (int)w, v.h = (int)h, v.image_index = (int)image_index, v.camera_index = (int)camera_index;
    v.camera_model_type = (int)camera_model_type;
    for (int i = 0; i < 5; ++i) v.crop_transform[i] = (float)crop_transform[i];
    for (int i = 0; i < 4; ++i) v.crop_rotation[i] = (float)crop_rotation[i];
    images.push_back(v);
}

void NeuralRenderInfo::clear_images() { images.clear(); }

void NeuralRenderInfo::set_params(int64_t num_layers_, int64_t k_keep, bool train_, bool drop_out_points_by_radius,
                                  double drop_out_radius_threshold, bool viewer_only, double stability_cutoff_value, bool bg_uses_Tn,
                                  double dropout_)
{
    num_layers = num_layers_, train = train_, dropout = dropout_;
    params.num_layers                = (int)num_layers_;
    params.k_keep                    = (int)k_keep;
    params.train                     = train_ ? 1 : 0;
    params.drop_out_points_by_radius = drop_out_points_by_radius ? 1 : 0;
    params.drop_out_radius_threshold = (float)drop_out_radius_threshold;
    params.viewer_only               = viewer_only ? 1 : 0;
    params.stability_cutoff_value    = (float)stability_cutoff_value;
    params.bg_uses_Tn                = bg_uses_Tn ? 1 : 0;
}

void NeuralRenderInfo::set_texture_preparation(bool confidence_is_raw, double confidence_scale, bool texture_abs)
{
    params.confidence_is_raw = confidence_is_raw ? 1 : 0;
    params.confidence_scale  = (float)confidence_scale;
    params.texture_abs       = texture_abs ? 1 : 0;
}

void NeuralRenderInfo::set_pipeline_flags(bool use_layer_point_size, bool render_points_in_all_lower_resolutions, bool combine_lists,
                                          bool saturated_alpha_accumulation)
{
    params.use_layer_point_size                   = use_layer_point_size ? 1 : 0;
    params.render_points_in_all_lower_resolutions = render_points_in_all_lower_resolutions ? 1 : 0;
    params.combine_lists                          = combine_lists ? 1 : 0;
    params.saturated_alpha_accumulation           = saturated_alpha_accumulation ? 1 : 0;
}

void NeuralRenderInfo::set_distortion(bool distortion, double dist_cutoff)
{
    params.distortion  = distortion ? 1 : 0;
    params.dist_cutoff = (float)dist_cutoff;
}

int64_t NeuralRenderInfo::last_status()
{
    return cache->handle ? (int64_t)trips_last_status(cache->handle, c10::cuda::getCurrentCUDAStream().stream()) : 0;
}

static const float* fptr(const Tensor& t) { return t.defined() ? t.data_ptr<float>() : nullptr; }

static void check_tensor(const Tensor& t, c10::ScalarType dt, const char* name)
{
    TORCH_CHECK(t.defined() && t.is_cuda() && t.is_contiguous() && t.scalar_type() == dt, name, " must be a contiguous CUDA tensor of the reference dtype");
}

static TripsScene make_scene(const NeuralRenderInfo& info, const Tensor& texture, const Tensor& background, const Tensor& points,
                             const Tensor& intrinsics, const Tensor& confidence, const Tensor& point_size)
{
    check_tensor(texture, torch::kFloat32, "texture");
    check_tensor(background, torch::kFloat32, "background_color");
    check_tensor(points, torch::kFloat32, "t_position");
    check_tensor(intrinsics, torch::kFloat32, "intrinsics");
    check_tensor(confidence, torch::kFloat32, "confidence_value_of_point");
    check_tensor(point_size, torch::kFloat32, "t_point_size");
    check_tensor(info.poses_se3, torch::kFloat64, "poses_se3");
    TORCH_CHECK(points.dim() == 2 && points.size(1) == 4 && intrinsics.size(1) == 13 && info.poses_se3.size(1) == 8,
                "expected t_position [N,4], intrinsics [n,13], poses_se3 [n,8]");
    TripsScene s{};
    s.n_points   = (int)points.size(0);
    s.n_tex      = (int)texture.size(1);
    s.channels   = (int)texture.size(0);
    s.position   = fptr(points);
    s.point_size = fptr(point_size);
    if (info.t_index.defined())
    {
        check_tensor(info.t_index, torch::kInt32, "t_index");
        s.index = info.t_index.data_ptr<int32_t>();
    }
    s.texture    = fptr(texture);
    s.confidence = fptr(confidence);
    s.background = fptr(background);
    s.dropout    = fptr(info.cache->dropout_points);
    s.poses      = info.poses_se3.data_ptr<double>();
    s.n_images   = (int)info.poses_se3.size(0);
    s.intrinsics = fptr(intrinsics);
    s.n_cameras  = (int)intrinsics.size(0);
    return s;
}

// PointRender (PointRenderer.h:39-47): forward = BlendPointCloudForward (PointRenderer.cu:676-1191), backward =
// BlendPointCloudBackward (PointRenderer.cu:1232-1427)
class PointRender : public torch::autograd::Function<PointRender>
{
   public:
    static torch::autograd::variable_list forward(torch::autograd::AutogradContext* ctx, Tensor texture, Tensor background_color,
                                                  Tensor points, Tensor pose_tangents, Tensor intrinsics, Tensor confidence,
                                                  Tensor dynamic_refinement, Tensor point_size, torch::IValue info_iv)
    {
        auto info = info_iv.toCustomClass<NeuralRenderInfo>();
        TORCH_CHECK(!info->images.empty(), "no images in the batch");
        TORCH_CHECK(!dynamic_refinement.defined() || dynamic_refinement.numel() == 0, "dynamic refinement is not implemented");
        TORCH_CHECK(points.is_cuda(), "the rasterizer runs on CUDA tensors only");
        auto& cache = *info->cache;
        cache.ensure(points.get_device());
        const int B = (int)info->images.size();
        cache.dropout_points = Tensor();
        if (info->train && info->dropout > 0)
            cache.dropout_points = torch::empty({B, points.size(0)}, points.options()).bernoulli_(info->dropout);
        TripsScene scene = make_scene(*info, texture, background_color, points, intrinsics, confidence, point_size);
        std::vector<Tensor> outs;
        std::vector<float*> out_ptrs;
        int w = info->images[0].w, h = info->images[0].h;
        for (int l = 0; l < info->num_layers; ++l)
        {
            outs.push_back(torch::empty({B, texture.size(0), h, w}, texture.options()));
            out_ptrs.push_back(outs.back().data_ptr<float>());
            w = (w + 1) / 2, h = (h + 1) / 2;  // ceil halving, PointRenderer.cu:385-389
        }
        TripsRenderParams params = info->params;
        params.num_layers        = (int)info->num_layers;
        params.train             = info->train ? 1 : 0;
        check(trips_forward(cache.handle, &scene, info->images.data(), B, &params, out_ptrs.data(), c10::cuda::getCurrentCUDAStream().stream()),
              cache.handle, "trips_forward");
        ctx->saved_data["info"] = info_iv;
        ctx->save_for_backward({texture, background_color, points, intrinsics, confidence, point_size, pose_tangents});
        return outs;
    }

    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list image_gradients)
    {
        auto info  = ctx->saved_data["info"].toCustomClass<NeuralRenderInfo>();
        auto saved = ctx->get_saved_variables();
        Tensor texture = saved[0], background = saved[1], points = saved[2], intrinsics = saved[3], confidence = saved[4], point_size = saved[5],
               pose_tangents = saved[6];
        auto& cache = *info->cache;
        std::vector<Tensor> keep;
        std::vector<const float*> gp;
        for (int l = 0; l < info->num_layers; ++l)
        {
            TORCH_CHECK(image_gradients[l].scalar_type() == torch::kFloat32, "image gradients must be float32");  // PointRenderer.cu:1236-1239
            keep.push_back(image_gradients[l].contiguous());
            gp.push_back(keep.back().data_ptr<float>());
        }
        Tensor g_tex = torch::empty_like(texture), g_bg = torch::empty_like(background), g_conf = torch::empty_like(confidence);
        Tensor g_pts, g_size, g_pose, g_intr;
        if (points.requires_grad()) g_pts = torch::empty_like(points);
        if (point_size.requires_grad()) g_size = torch::empty_like(point_size);
        if (pose_tangents.defined() && pose_tangents.requires_grad())
            g_pose = torch::empty({info->poses_se3.size(0), 6}, info->poses_se3.options());
        if (intrinsics.requires_grad()) g_intr = torch::empty_like(intrinsics);
        TripsGrads g{g_tex.data_ptr<float>(), g_bg.data_ptr<float>(), g_pts.defined() ? g_pts.data_ptr<float>() : nullptr,
                     g_pose.defined() ? g_pose.data_ptr<double>() : nullptr, g_intr.defined() ? g_intr.data_ptr<float>() : nullptr,
                     g_conf.data_ptr<float>(), g_size.defined() ? g_size.data_ptr<float>() : nullptr};
        TripsScene scene = make_scene(*info, texture, background, points, intrinsics, confidence, point_size);
        check(trips_backward(cache.handle, &scene, gp.data(), &g, c10::cuda::getCurrentCUDAStream().stream()), cache.handle, "trips_backward");
        // order of PointRenderer.cu:1423-1426: texture, background, points, pose tangents, intrinsics, confidence,
        // dynamic refinement (undefined), point size; plus one empty Variable for the info argument (RenderInfo.cpp:77)
        return {g_tex, g_bg, g_pts, g_pose, g_intr, g_conf, Tensor(), g_size, Tensor()};
    }
};

std::vector<Tensor> BlendPointCloud(const c10::intrusive_ptr<NeuralRenderInfo>& info)
{
    TORCH_CHECK(info->texture.defined() && info->t_position.defined(), "NeuralRenderInfo has no scene");
    const Tensor tangents = info->tangent_poses.defined() ? info->tangent_poses : torch::empty({0}, info->poses_se3.options());
    return PointRender::apply(info->texture, info->background_color, info->t_position, tangents, info->intrinsics,
                              info->confidence_value_of_point, torch::empty({0}, info->t_position.options()) /* dynamic refinement: none */,
                              info->t_point_size, torch::IValue(info));
}

PointRenderModuleImpl::PointRenderModuleImpl(int num_layers_) : num_layers(num_layers_), cache(std::make_shared<PointRendererCache>()) {}

std::pair<std::vector<Tensor>, std::vector<Tensor>> PointRenderModuleImpl::forward(const c10::intrusive_ptr<NeuralRenderInfo>& nri)
{
    nri->cache      = cache;  // RenderModule.cpp:57
    nri->num_layers = num_layers;
    if (!is_training())  // RenderModule.cpp:27-35
    {
        nri->dropout = 0;
        nri->train   = false;
    }
    else
        nri->train = true;
    auto images = BlendPointCloud(nri);
    images.resize(num_layers);
    return {images, {}};
}

// ------------------------------------------------------------------------------------------------------------
// MyAdam
// ------------------------------------------------------------------------------------------------------------
MyAdam::MyAdam(std::vector<torch::optim::OptimizerParamGroup> param_groups, MyAdamOptions defaults)
    : Optimizer(std::move(param_groups), std::make_unique<MyAdamOptions>(defaults))
{
    TORCH_CHECK(defaults.lr() >= 0, "Invalid learning rate: ", defaults.lr());
    TORCH_CHECK(defaults.eps() >= 0, "Invalid epsilon value: ", defaults.eps());
    auto betas = defaults.betas();
    TORCH_CHECK(0 <= std::get<0>(betas) && std::get<0>(betas) < 1.0, "Invalid beta parameter at index 0: ", std::get<0>(betas));
    TORCH_CHECK(0 <= std::get<1>(betas) && std::get<1>(betas) < 1.0, "Invalid beta parameter at index 1: ", std::get<1>(betas));
    TORCH_CHECK(defaults.relative_weight_decay() >= 0, "Invalid relative_weight_decay value: ", defaults.relative_weight_decay());
    TORCH_CHECK(defaults.absolute_weight_decay() >= 0, "Invalid absolute_weight_decay value: ", defaults.absolute_weight_decay());
}

MyAdam::MyAdam(std::vector<Tensor> params, MyAdamOptions defaults)
    : MyAdam(std::vector<torch::optim::OptimizerParamGroup>{torch::optim::OptimizerParamGroup(std::move(params))}, defaults)
{
}

MyAdam::~MyAdam()
{
    if (ctx_) trips_context_destroy(ctx_);
}

MyAdamParamState* MyAdam::state_of(const Tensor& p)
{
    auto it = state_.find(p.unsafeGetTensorImpl());
    return it == state_.end() ? nullptr : static_cast<MyAdamParamState*>(it->second.get());
}

Tensor MyAdam::step(LossClosure closure)
{
    torch::NoGradGuard no_grad;
    Tensor loss = {};
    if (closure != nullptr)
    {
        at::AutoGradMode enable_grad(true);
        loss = closure();
    }
    std::vector<TripsAdamTensor> table;
    std::vector<Tensor> keep;  // contiguous gradients stay alive until the launch is enqueued
    for (auto& group : param_groups_)
    {
        auto& options = static_cast<MyAdamOptions&>(group.options());
        for (auto& p : group.params())
        {
            if (!p.grad().defined()) continue;
            auto grad = p.grad();
            TORCH_CHECK(!grad.is_sparse(), "Adam does not support sparse gradients");
            TORCH_CHECK(p.scalar_type() == torch::kFloat32 && p.is_cuda() && p.is_contiguous(), "MyAdam takes contiguous float32 CUDA parameters");
            if (device_ != p.get_device())
            {
                TORCH_CHECK(device_ < 0, "all parameters of one MyAdam must live on one device");
                device_ = p.get_device();
                check(trips_context_create(&ctx_, device_), nullptr, "trips_context_create");
            }
            MyAdamParamState* st = state_of(p);
            if (!st)  // state initialisation, MyAdam.cu:184-200
            {
                auto state = std::make_unique<MyAdamParamState>();
                state->param_steps(torch::zeros(p.sizes(), p.options().dtype(torch::kInt32)));
                state->first_moments(torch::zeros_like(p, torch::MemoryFormat::Contiguous));
                state->second_moments(torch::zeros_like(p, torch::MemoryFormat::Contiguous));
                state->current_step(0);
                st                                = state.get();
                state_[p.unsafeGetTensorImpl()] = std::move(state);
            }
            st->current_step(st->current_step() + 1);
            const float beta1 = (float)std::get<0>(options.betas()), beta2 = (float)std::get<1>(options.betas());
            float lower = 0.f, upper = std::numeric_limits<float>::max();
            if (options.adabound())  // MyAdam.cu:220-224
            {
                lower = 0.1f - 0.1f / ((1 - beta2) * (float)st->current_step() + 1);
                upper = 0.1f + 0.1f / ((1 - beta2) * (float)st->current_step());
            }
            keep.push_back(grad.contiguous());
            TORCH_CHECK(keep.back().scalar_type() == torch::kFloat32 && keep.back().numel() == p.numel(), "gradient must match the parameter");
            table.push_back(TripsAdamTensor{p.data_ptr<float>(), keep.back().data_ptr<float>(), st->first_moments().data_ptr<float>(),
                                            st->second_moments().data_ptr<float>(), st->param_steps().data_ptr<int32_t>(), p.numel(),
                                            (float)options.lr(), beta1, beta2, (float)options.eps(), (float)options.relative_weight_decay(),
                                            (float)options.absolute_weight_decay(), (float)options.weight_clipping_magnitude(), lower, upper});
        }
    }
    if (!table.empty())
        check(trips_adam_step(ctx_, table.data(), (int)table.size(), c10::cuda::getCurrentCUDAStream(device_).stream()), ctx_, "trips_adam_step");
    return loss;
}

void MyAdam::save(torch::serialize::OutputArchive&) const { TORCH_CHECK(false, "MyAdam::save is not supported (as in the reference)"); }
void MyAdam::load(torch::serialize::InputArchive&) { TORCH_CHECK(false, "MyAdam::load is not supported (as in the reference)"); }

void MyAdam::shrinkInternalState(int param_group_index, Tensor indices_to_keep)
{
    TORCH_CHECK(param_group_index >= 0 && param_group_index < (int)param_groups_.size(), "param group out of range");
    torch::NoGradGuard no_grad;
    for (auto& p : param_groups_[param_group_index].params())
    {
        MyAdamParamState* st = state_of(p);
        if (!st) continue;  // not created yet: initialised by the first step
        auto shrink = [&](Tensor t) {
            return t.index_select(t.dim() - 1, indices_to_keep.reshape({-1}).to(t.device()).to(torch::kLong)).contiguous();
        };
        st->first_moments(shrink(st->first_moments()));
        st->second_moments(shrink(st->second_moments()));
        st->param_steps(shrink(st->param_steps()));
    }
}

void MyAdam::appendToInternalState(int param_group_index, int new_size)
{
    TORCH_CHECK(param_group_index >= 0 && param_group_index < (int)param_groups_.size(), "param group out of range");
    torch::NoGradGuard no_grad;
    for (auto& p : param_groups_[param_group_index].params())
    {
        MyAdamParamState* st = state_of(p);
        if (!st) continue;
        auto extend = [&](Tensor t) {
            std::vector<int64_t> sizes(t.sizes().begin(), t.sizes().end());
            sizes.back() = new_size - t.size(-1);
            TORCH_CHECK(sizes.back() >= 0, "appendToInternalState cannot shrink");
            return torch::cat({t, torch::zeros(sizes, t.options())}, -1).contiguous();
        };
        st->first_moments(extend(st->first_moments()));
        st->second_moments(extend(st->second_moments()));
        st->param_steps(extend(st->param_steps()));
    }
}

void UpdateOptimLR(torch::optim::Optimizer* optimizer, double factor)
{
    for (auto& pg : optimizer->param_groups()) pg.options().set_lr(pg.options().get_lr() * factor);
}

// ------------------------------------------------------------------------------------------------------------
// parameter modules (registered names = checkpoint format)
// ------------------------------------------------------------------------------------------------------------
NeuralPointCloudCudaImpl::NeuralPointCloudCudaImpl(Tensor position, Tensor point_size, Tensor index, Tensor original_color)
{
    t_position       = register_parameter("t_position", position);
    t_index          = register_buffer("t_index", index);
    t_original_color = register_buffer("t_original_color", original_color);
    t_point_size     = register_parameter("t_point_size", point_size);
}

NeuralPointTextureImpl::NeuralPointTextureImpl(int num_channels, int num_points)
{
    texture_raw          = register_parameter("texture", torch::ones({num_channels, num_points}) * 0.5);
    background_color_raw = register_parameter("background_color", torch::ones({num_channels}) * 0.25);
    confidence_raw       = register_parameter("confidence_value_of_point", torch::ones({1, num_points}) * 0.5);
}

PoseModuleImpl::PoseModuleImpl(int num_images)
{
    tangent_poses = register_parameter("tangent_poses", torch::zeros({num_images, 6}, torch::kFloat64));
    poses_se3     = register_buffer("poses_se3", torch::zeros({num_images, 8}, torch::kFloat64));
}

IntrinsicsModuleImpl::IntrinsicsModuleImpl(int num_cameras)
{
    intrinsics = register_parameter("intrinsics", torch::zeros({num_cameras, 13}));
}

// ------------------------------------------------------------------------------------------------------------
// registration for Python (tests drive the C++ classes through these)
// ------------------------------------------------------------------------------------------------------------
namespace
{
struct PointRenderModuleHolder : torch::CustomClassHolder
{
    PointRenderModule module;
    explicit PointRenderModuleHolder(int64_t num_layers) : module((int)num_layers) {}
    void train(bool on) { module->train(on); }
    std::vector<Tensor> forward(const c10::intrusive_ptr<NeuralRenderInfo>& nri) { return module->forward(nri).first; }
};

struct MyAdamHolder : torch::CustomClassHolder
{
    std::unique_ptr<MyAdam> opt;
    void add_param_group(std::vector<Tensor> params, double lr, double beta1, double beta2, double eps, double relative_weight_decay,
                         double absolute_weight_decay, double weight_clipping_magnitude, bool adabound)
    {
        MyAdamOptions o(lr);
        o.betas(std::make_tuple(beta1, beta2)).eps(eps).relative_weight_decay(relative_weight_decay).absolute_weight_decay(absolute_weight_decay);
        o.weight_clipping_magnitude(weight_clipping_magnitude).adabound(adabound);
        torch::optim::OptimizerParamGroup g(std::move(params), std::make_unique<MyAdamOptions>(o));
        if (!opt)
            opt = std::make_unique<MyAdam>(std::vector<torch::optim::OptimizerParamGroup>{g}, o);
        else
            opt->add_param_group(g);
    }
    void step()
    {
        TORCH_CHECK(opt, "no param group");
        opt->step();
    }
    void shrinkInternalState(int64_t group, Tensor keep) { opt->shrinkInternalState((int)group, keep); }
    void appendToInternalState(int64_t group, int64_t new_size) { opt->appendToInternalState((int)group, (int)new_size); }
    void scale_lr(double factor) { UpdateOptimLR(opt.get(), factor); }
    // (first_moments, second_moments, param_steps) of parameter `index` of `group`; empty before its first step
    std::vector<Tensor> state(int64_t group, int64_t index)
    {
        auto* st = opt->state_of(opt->param_groups().at(group).params().at(index));
        if (!st) return {};
        return {st->first_moments(), st->second_moments(), st->param_steps()};
    }
};

// One context per device for the functional adam_step operator below.
TripsContext* functional_context(int device)
{
    static std::mutex mu;
    static TripsContext* ctx[64] = {};
    std::lock_guard<std::mutex> lock(mu);
    TORCH_CHECK(device >= 0 && device < 64, "device index out of range");
    if (!ctx[device]) check(trips_context_create(&ctx[device], device), nullptr, "trips_context_create");
    return ctx[device];
}
}  // namespace

// MyAdam::step over explicit lists of tensors, for callers that keep the optimizer state themselves (MyAdam.cu:164-345
// launches adam_step once per tensor; here one launch covers all of them).  State tensors: first_moments,
// second_moments (float32, shape of the parameter) and param_steps (int32 here, int64 in the reference).  Runs through
// trips_adam_step on a context the library keeps per device: calls on one device are ordered by their streams as usual.
void AdamStep(std::vector<Tensor> weights, std::vector<Tensor> gradients, std::vector<Tensor> first_moments,
              std::vector<Tensor> second_moments, std::vector<Tensor> steps, double lr, double beta1, double beta2, double eps)
{
    const size_t n = weights.size();
    TORCH_CHECK(n > 0, "no tensors");
    TORCH_CHECK(gradients.size() == n && first_moments.size() == n && second_moments.size() == n && steps.size() == n,
                "one gradient and one state triple per weight tensor");
    std::vector<TripsAdamTensor> table(n);
    for (size_t i = 0; i < n; ++i)
    {
        check_tensor(weights[i], torch::kFloat32, "weights");
        check_tensor(gradients[i], torch::kFloat32, "gradients");
        check_tensor(first_moments[i], torch::kFloat32, "first_moments");
        check_tensor(second_moments[i], torch::kFloat32, "second_moments");
        check_tensor(steps[i], torch::kInt32, "param_steps");
        const int64_t k = weights[i].numel();
        TORCH_CHECK(gradients[i].numel() == k && first_moments[i].numel() == k && second_moments[i].numel() == k && steps[i].numel() == k,
                    "gradient and state must have the parameter's size");
        table[i] = TripsAdamTensor{weights[i].data_ptr<float>(), gradients[i].data_ptr<float>(), first_moments[i].data_ptr<float>(),
                                   second_moments[i].data_ptr<float>(), steps[i].data_ptr<int32_t>(), k, (float)lr, (float)beta1, (float)beta2,
                                   (float)eps, 0.f, 0.f, 0.f, 0.f, 3.4028234663852886e38f};
    }
    const int device  = weights[0].get_device();
    TripsContext* ctx = functional_context(device);
    check(trips_adam_step(ctx, table.data(), (int)n, c10::cuda::getCurrentCUDAStream(device).stream()), ctx, "trips_adam_step");
}

TORCH_LIBRARY(trips_b200, m)
{
    m.class_<NeuralRenderInfo>("NeuralRenderInfo")
        .def(torch::init<>())
        .def("set_scene", &NeuralRenderInfo::set_scene)
        .def("add_image", &NeuralRenderInfo::add_image)
        .def("clear_images", &NeuralRenderInfo::clear_images)
        .def("set_params", &NeuralRenderInfo::set_params)
        .def("set_texture_preparation", &NeuralRenderInfo::set_texture_preparation)
        .def("set_pipeline_flags", &NeuralRenderInfo::set_pipeline_flags)
        .def("set_distortion", &NeuralRenderInfo::set_distortion)
        .def("last_status", &NeuralRenderInfo::last_status);
    m.class_<PointRenderModuleHolder>("PointRenderModule")
        .def(torch::init<int64_t>())
        .def("train", &PointRenderModuleHolder::train)
        .def("forward", &PointRenderModuleHolder::forward);
    m.class_<MyAdamHolder>("MyAdam")
        .def(torch::init<>())
        .def("add_param_group", &MyAdamHolder::add_param_group)
        .def("step", &MyAdamHolder::step)
        .def("shrinkInternalState", &MyAdamHolder::shrinkInternalState)
        .def("appendToInternalState", &MyAdamHolder::appendToInternalState)
        .def("scale_lr", &MyAdamHolder::scale_lr)
        .def("state", &MyAdamHolder::state);
    m.def("blend_point_cloud(__torch__.torch.classes.trips_b200.NeuralRenderInfo info) -> Tensor[]", &BlendPointCloud);
    m.def("adam_step(Tensor[] weights, Tensor[] gradients, Tensor[] first_moments, Tensor[] second_moments, Tensor[] steps, float lr, "
          "float beta1, float beta2, float eps) -> ()",
          &AdamStep);
}
}  // namespace trips_b200
