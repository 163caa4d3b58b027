// Reads the four module archives of a checkpoint with libtorch (torch::load into modules that register the reference's
// tensor names, as NeuralScene::LoadCheckpoint does, src/lib/data/NeuralScene.cpp:533-590), prints a checksum per
// tensor, and writes them back with torch::save (NeuralScene::SaveCheckpoint, :595-628) under another prefix.
// Compiled and run by tests/test_checkpoint.py; CPU only.
#include <cstdio>
#include <cstdlib>
#include <string>

#include "torch_shim.h"

static void report(const char* name, const torch::Tensor& t)
{
    std::printf("%s %s %lld %.17g\n", name, c10::toString(t.scalar_type()), (long long)t.numel(), t.to(torch::kFloat64).sum().item<double>());
}

int main(int argc, char** argv)
{
    if (argc != 7) return 2;
    using namespace trips_b200;
    const std::string in = argv[1], out = argv[6];
    const int N = std::atoi(argv[2]), C = std::atoi(argv[3]), n_images = std::atoi(argv[4]), n_cameras = std::atoi(argv[5]);
    NeuralPointCloudCuda pc(torch::zeros({N, 4}), torch::zeros({N, 1}), torch::zeros({N, 1}, torch::kInt32), torch::zeros({N, 4}));
    NeuralPointTexture tex(C, N);
    PoseModule poses(n_images);
    IntrinsicsModule intr(n_cameras);
    torch::load(pc, in + "points.pth");
    torch::load(tex, in + "texture.pth", torch::kCPU);
    torch::load(poses, in + "poses.pth");
    torch::load(intr, in + "intrinsics.pth");
    report("t_position", pc->t_position);
    report("t_point_size", pc->t_point_size);
    report("t_index", pc->t_index);
    report("t_original_color", pc->t_original_color);
    report("texture", tex->texture_raw);
    report("background_color", tex->background_color_raw);
    report("confidence_value_of_point", tex->confidence_raw);
    report("tangent_poses", poses->tangent_poses);
    report("poses_se3", poses->poses_se3);
    report("intrinsics", intr->intrinsics);
    torch::save(pc, out + "points.pth");
    torch::save(tex, out + "texture.pth");
    torch::save(poses, out + "poses.pth");
    torch::save(intr, out + "intrinsics.pth");
    return 0;
}
