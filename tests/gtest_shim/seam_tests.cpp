// Tests of what the B200 seams add to ormi-core (own cases, not the reference's): a lowering registered through the
// reference's plug-in point reaches the generated CUDA code, and graphs run on the device that owns their inputs.
#include <gtest/gtest.h>

#include <cmath>
#include <memory>
#include <string>
#include <vector>

#include "tests/test_utils.h"
#include "core/memory.h"
#include "core/node.h"
#include "core/ops.h"
#include "core/ops/pointwise/add.h"
#include "core/ops/pointwise/sin.h"
#include "backend/runtime.h"
#include "backend/cuda/compiler.cuh"
#include "backend/cuda/jit.cuh"
#include "backend/cuda/lowering_registry.h"
#include "b200_backend.h"

using namespace ormi;

namespace {
using Names = const std::vector<std::string>&;

struct RestoreSin {      // the registry is process-wide: put the stock lowering back whatever the test does
    ~RestoreSin() { cuda::CUDALoweringRegistry::register_func(ops::OpEnum::SIN, [](Names o) { return "sinf(" + o[0] + ");"; }); }
};

std::shared_ptr<Node> leaf(const std::vector<int>& shape, float v, DeviceEnum dev) {
    return std::make_shared<Node>(full(shape, v, dev), false, Device(dev));
}
}  // namespace

class B200SeamTest : public ormi::testing::HardwareTestSuite {
protected:
    bool has_cuda = false;
    void SetUp() override {
        HardwareTestSuite::SetUp();
        for (auto d : available_devices) has_cuda |= d == DeviceEnum::CUDA;
    }
};

TEST_F(B200SeamTest, RegisteredLoweringShowsInCompiledSource) {
    RestoreSin restore;
    auto x = leaf({4}, 0.0f, DeviceEnum::CPU);                 // compile() only reads shapes: no device needed
    x->device = Device(DeviceEnum::CUDA);
    auto y = ops::sin(x);
    EXPECT_NE(cuda::compile(y).kernel_code.find("sinf("), std::string::npos);
    cuda::CUDALoweringRegistry::register_func(ops::OpEnum::SIN, [](Names o) { return "cosf(" + o[0] + ") * 2.0f;"; });
    const std::string code = cuda::compile(ops::sin(x)).kernel_code;
    EXPECT_NE(code.find("cosf("), std::string::npos);
    EXPECT_EQ(code.find("sinf("), std::string::npos);
}

TEST_F(B200SeamTest, RegisteredLoweringRunsOnCuda) {
    if (!has_cuda) GTEST_SKIP() << "CUDA device unavailable";
    RestoreSin restore;
    auto x = leaf({2, 1024}, 0.0f, DeviceEnum::CUDA);
    auto run = [&]() {
        auto y = ops::add(ops::sin(x), x);                     // a fused kernel, not a lone node
        execute_graph(y);
        std::vector<float> out(2048);
        get_allocator(DeviceEnum::CUDA)->copy_device_to_host(out.data(), y->data->ptr, out.size() * sizeof(float));
        return out;
    };
    for (float v : run()) EXPECT_FLOAT_EQ(v, 0.0f);            // sin(0) + 0
    cuda::CUDALoweringRegistry::register_func(ops::OpEnum::SIN, [](Names o) { return "cosf(" + o[0] + ") * 2.0f;"; });
    for (float v : run()) EXPECT_FLOAT_EQ(v, 2.0f);            // the registered expression: cos(0) * 2 + 0
    cuda::CUDALoweringRegistry::register_func(ops::OpEnum::SIN, [](Names o) { return "sinf(" + o[0] + ");"; });
    for (float v : run()) EXPECT_FLOAT_EQ(v, 0.0f);            // and the stock one again: the cached schedule was not reused
}

TEST_F(B200SeamTest, GraphsRunOnTheDeviceThatOwnsTheirInputs) {
    if (!has_cuda) GTEST_SKIP() << "CUDA device unavailable";
    EXPECT_EQ(cuda::active_device(), 0);
    EXPECT_NE(cuda::b200_context(), nullptr);
    EXPECT_THROW(cuda::set_active_device(4096), std::runtime_error);      // no such device: refused, active device unchanged
    EXPECT_EQ(cuda::active_device(), 0);
    auto a = leaf({8}, 1.5f, DeviceEnum::CUDA);
    auto y = ops::add(a, a);
    y->device = Device(DeviceEnum::CUDA, 3);                              // placed elsewhere than its inputs live
    EXPECT_THROW(execute_graph(y), std::runtime_error);
    auto z = ops::add(a, a);
    execute_graph(z);
    std::vector<float> out(8);
    get_allocator(DeviceEnum::CUDA)->copy_device_to_host(out.data(), z->data->ptr, out.size() * sizeof(float));
    for (float v : out) EXPECT_FLOAT_EQ(v, 3.0f);
}
