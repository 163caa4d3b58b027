// libtorch host side of the rasterizer: the reference's operator interface on top of the C ABI.
//
// Same names and argument order as the reference (src/lib/rendering/PointRenderer.h:23-53, RenderInfo.cpp:14-40):
// NeuralRenderInfo (a torch custom class), PointRendererCache, torch::autograd::PointRender and BlendPointCloud.  The
// reference reaches its tensors through NeuralScene modules; here the info object holds the same tensors directly
// (texture, background_color, t_position, poses_se3, intrinsics, confidence_value_of_point, t_point_size, t_index).
// Tensors are flattened to device pointers and handed to trips_forward / trips_backward on the current CUDA stream;
// nothing is computed in this file.  Registered as torch.classes.trips_b200.NeuralRenderInfo,
// torch.ops.trips_b200.blend_point_cloud and torch.ops.trips_b200.adam_step (MyAdam::step), which is how tests/ drive it.
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/torch.h>

#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "trips_b200.h"

namespace trips_shim
{
using torch::Tensor;

// owns the C context, like PointRendererCache owns the reference's scratch tensors (PointRenderer.h:126-176)
struct PointRendererCache
{
    TripsContext* handle = nullptr;
    int device           = -1;
    Tensor dropout_points;  // [B,N], training with dropout > 0 only (PointRenderer.cu:518-523)
    ~PointRendererCache()
    {
        if (handle) trips_context_destroy(handle);
    }
    void ensure(int dev)
    {
        if (handle && dev == device) return;
        if (handle) trips_context_destroy(handle);
        handle = nullptr;
        const int st = trips_context_create(&handle, dev);
        if (st != TRIPS_OK) throw std::runtime_error(std::string("trips_context_create: ") + trips_status_string(st));
        device = dev;
    }
};

static void check(int st, TripsContext* ctx, const char* what)
{
    if (st != TRIPS_OK) throw std::runtime_error(std::string(what) + ": " + trips_status_string(st) + " (" + trips_last_error(ctx) + ")");
}

struct NeuralRenderInfo : torch::CustomClassHolder
{
    // scene (NeuralScene: point_cloud_cuda, texture, poses, intrinsics)
    Tensor texture, background_color, t_position, poses_se3, intrinsics, confidence_value_of_point, t_point_size, t_index;
    std::vector<TripsView> images;  // ReducedImageInfo, SceneData.h:40-61
    TripsRenderParams params{8, 16, 0, 0, 0.f, 0, 0.f, 0};
    double dropout = 0.0;
    int64_t num_layers = 8;
    bool train         = false;
    std::shared_ptr<PointRendererCache> cache = std::make_shared<PointRendererCache>();

    void set_scene(Tensor texture_, Tensor background_color_, Tensor t_position_, Tensor poses_se3_, Tensor intrinsics_,
                   Tensor confidence_, Tensor t_point_size_, c10::optional<Tensor> t_index_)
    {
        texture = texture_, background_color = background_color_, t_position = t_position_, poses_se3 = poses_se3_;
        intrinsics = intrinsics_, confidence_value_of_point = confidence_, t_point_size = t_point_size_;
        t_index = t_index_.has_value() ? *t_index_ : Tensor();
    }
    void add_image(int64_t w, int64_t h, int64_t image_index, int64_t camera_index, int64_t camera_model_type,
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
    void clear_images() { images.clear(); }
    void set_params(int64_t num_layers_, int64_t k_keep, bool train_, bool drop_out_points_by_radius, double drop_out_radius_threshold,
                    bool viewer_only, double stability_cutoff_value, bool bg_uses_Tn, double dropout_)
    {
        num_layers = num_layers_, train = train_, dropout = dropout_;
        params = TripsRenderParams{(int)num_layers_, (int)k_keep, train_ ? 1 : 0, drop_out_points_by_radius ? 1 : 0,
                                   (float)drop_out_radius_threshold, viewer_only ? 1 : 0, (float)stability_cutoff_value, bg_uses_Tn ? 1 : 0};
    }
    int64_t last_status() { return cache->handle ? (int64_t)trips_last_status(cache->handle, c10::cuda::getCurrentCUDAStream().stream()) : 0; }
};

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

// BlendPointCloud (RenderInfo.cpp:27-40)
std::vector<Tensor> BlendPointCloud(const c10::intrusive_ptr<NeuralRenderInfo>& info, const Tensor& pose_tangents)
{
    return PointRender::apply(info->texture, info->background_color, info->t_position, pose_tangents, info->intrinsics,
                              info->confidence_value_of_point, torch::empty({0}, info->t_position.options()) /* dynamic refinement: none */,
                              info->t_point_size, torch::IValue(info));
}

// MyAdam::step over a list of parameter tensors (MyAdam.cu:164-345 launches adam_step once per tensor; here one launch
// covers all of them).  State tensors are those MyAdam keeps per parameter: first_moments, second_moments (float32,
// shape of the parameter) and param_steps (int32 here, int64 in the reference).  Updates weights and state in place.
void AdamStep(std::vector<Tensor> weights, std::vector<Tensor> gradients, std::vector<Tensor> first_moments,
              std::vector<Tensor> second_moments, std::vector<Tensor> steps, double lr, double beta1, double beta2, double eps)
{
    const size_t n = weights.size();
    TORCH_CHECK(n > 0 && n <= TRIPS_ADAM_STATIC_MAX_TENSORS, "1 to ", TRIPS_ADAM_STATIC_MAX_TENSORS, " tensors per call");
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
    const int st = trips_adam_step_static(table.data(), (int)n, c10::cuda::getCurrentCUDAStream().stream());
    TORCH_CHECK(st == TRIPS_OK, "trips_adam_step_static: ", trips_status_string(st));
}

TORCH_LIBRARY(trips_b200, m)
{
    m.class_<NeuralRenderInfo>("NeuralRenderInfo")
        .def(torch::init<>())
        .def("set_scene", &NeuralRenderInfo::set_scene)
        .def("add_image", &NeuralRenderInfo::add_image)
        .def("clear_images", &NeuralRenderInfo::clear_images)
        .def("set_params", &NeuralRenderInfo::set_params)
        .def("last_status", &NeuralRenderInfo::last_status);
    m.def("blend_point_cloud(__torch__.torch.classes.trips_b200.NeuralRenderInfo info, Tensor pose_tangents) -> Tensor[]", &BlendPointCloud);
    m.def("adam_step(Tensor[] weights, Tensor[] gradients, Tensor[] first_moments, Tensor[] second_moments, Tensor[] steps, float lr, "
          "float beta1, float beta2, float eps) -> ()",
          &AdamStep);
}
}  // namespace trips_shim
