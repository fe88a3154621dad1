// torch.ops.dandan_ops.* over the C ABI: the operator surface the reference registers from C++
// (dandan_ops/csrc/operators.cu:259-278, dandan_ops/csrc/hgemm.cu:89-98) and loads with
// torch.ops.load_library (dandan_ops/_extension.py:34), here as a thin layer that validates tensors,
// allocates the output and the workspace through ATen and forwards to libb2w4a16.so on the current
// CUDA stream.  The four reference op names run the one engine; they differ only in the argument
// rule each reference op enforces.  `w4a16_linear_image` is the entry the Python module uses per
// token: it takes the device-native image directly, so no cache lookup sits on the hot path.
//
// Nothing here computes: a missing or failing C-ABI call raises.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <climits>
#include <mutex>
#include <tuple>
#include <unordered_map>
#include <vector>

#include "../../../include/b2_w4a16.h"

namespace {

std::mutex g_mutex;

// ---- workspaces: one per (device, stream), grown geometrically, never released -----------------
// A CUDA graph captured earlier keeps the raw address of the workspace it was captured with, so a
// buffer that a kernel has seen stays allocated for the life of the process.
struct Pool {
    std::unordered_map<uint64_t, at::Tensor> live;
    std::vector<at::Tensor> retired;
};
Pool& pool() {
    static Pool* p = new Pool();      // never destroyed: tensors must not be freed after CUDA shuts down
    return *p;
}

at::Tensor workspace_for(const at::Device& device, cudaStream_t stream, int64_t need) {
    const uint64_t key = (uint64_t(device.index()) << 56) ^ reinterpret_cast<uint64_t>(stream);
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = pool().live.find(key);
    if (it != pool().live.end() && it->second.numel() >= need) return it->second;
    int64_t size = std::max<int64_t>(need, 1 << 20);
    if (it != pool().live.end()) {
        size = std::max(size, 2 * it->second.numel());
        pool().retired.push_back(it->second);
    }
    at::Tensor fresh = at::zeros({size}, at::TensorOptions().dtype(at::kByte).device(device));
    pool().live[key] = fresh;
    return fresh;
}

void check_rc(int rc) {
    TORCH_CHECK(rc == B2_OK, "b2_w4a16: ", b2_w4a16_last_error());
}

// ---- native images of reference-layout state, for the four legacy ops ---------------------------
struct ImageEntry {
    c10::weak_intrusive_ptr<c10::TensorImpl> owner;
    std::tuple<void*, void*, void*, uint32_t, uint32_t, uint32_t, int64_t, int64_t> stamp;
    at::Tensor image;
};
std::unordered_map<void*, ImageEntry>& images() {
    static auto* m = new std::unordered_map<void*, ImageEntry>();
    return *m;
}

at::Tensor image_for(const at::Tensor& packed, const at::Tensor& scales, const at::Tensor& zeros, int64_t k) {
    const auto stamp = std::make_tuple(packed.data_ptr(), scales.data_ptr(), zeros.data_ptr(), packed._version(),
                                       scales._version(), zeros._version(), packed.size(0), k);
    void* id = packed.unsafeGetTensorImpl();
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        auto it = images().find(id);
        if (it != images().end() && !it->second.owner.expired() && it->second.stamp == stamp) return it->second.image;
        for (auto e = images().begin(); e != images().end();)            // drop entries whose tensors are gone
            e = e->second.owner.expired() ? images().erase(e) : std::next(e);
    }
    const int64_t bytes = b2_w4a16_native_bytes(packed.size(0), k);
    TORCH_CHECK(bytes > 0, "W4A16 dimensions exceed the kernel index range");
    at::Tensor image = at::empty({bytes}, packed.options().dtype(at::kByte));
    check_rc(b2_w4a16_repack(packed.data_ptr<int32_t>(), scales.data_ptr<float>(), zeros.data_ptr<int32_t>(), packed.size(0), k,
                             image.data_ptr(), at::cuda::getCurrentCUDAStream().stream()));
    std::lock_guard<std::mutex> lock(g_mutex);
    images().erase(id);
    images().emplace(id, ImageEntry{c10::weak_intrusive_ptr<c10::TensorImpl>(packed.getIntrusivePtr()), stamp, image});
    return image;
}

// ---- argument checks of the reference's native ops (dandan_ops/csrc/gemm_checks.h:6-30) --------
void check_w4a16(const at::Tensor& x, const at::Tensor& packed, const at::Tensor& scales, const at::Tensor& zeros,
                 int64_t group_size) {
    const at::Tensor* all[4] = {&x, &packed, &scales, &zeros};
    bool two_d = true, cuda = true, same = true, dense = true;
    for (const at::Tensor* t : all) {
        two_d = two_d && t->dim() == 2;
        cuda = cuda && t->is_cuda();
        same = same && t->device() == x.device();
        dense = dense && t->is_contiguous();
    }
    TORCH_CHECK(two_d, "W4A16 tensors must be 2D");
    TORCH_CHECK(cuda, "W4A16 expects CUDA tensors");
    TORCH_CHECK(same, "W4A16 tensors must share a device");
    TORCH_CHECK(x.scalar_type() == at::kHalf && packed.scalar_type() == at::kInt && scales.scalar_type() == at::kFloat &&
                    zeros.scalar_type() == at::kInt, "invalid W4A16 dtypes");
    TORCH_CHECK(dense, "W4A16 tensors must be contiguous");
    const int64_t m = x.size(0), k = x.size(1), n = packed.size(0);
    TORCH_CHECK(k > 0 && n > 0 && k <= INT_MAX - 64 && n <= INT_MAX - 64 && m <= INT_MAX - 128, "invalid W4A16 dimensions");
    TORCH_CHECK(group_size > 0 && group_size <= INT_MAX - k, "invalid group_size");
    TORCH_CHECK(x.numel() <= INT_MAX && m * n <= INT_MAX && n * k <= INT_MAX, "W4A16 dimensions exceed the kernel index range");
    TORCH_CHECK(packed.size(1) == (k + 7) / 8, "invalid packed weight shape");
    const int64_t groups = (k + group_size - 1) / group_size;
    TORCH_CHECK(scales.size(0) == n && scales.size(1) == groups && zeros.sizes() == scales.sizes(), "invalid W4A16 metadata shape");
}

at::Tensor run_image(const at::Tensor& x, const at::Tensor& image, int64_t n, int64_t k, const c10::optional<at::Tensor>& bias,
                     int64_t route, int64_t flags = 0) {
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t m = x.size(0);
    at::Tensor y = at::empty({m, n}, x.options());
    if (m == 0) return y;
    cudaStream_t stream = at::cuda::getCurrentCUDAStream().stream();
    at::Tensor ws = workspace_for(x.device(), stream, b2_w4a16_workspace_bytes(m, n, k));
    const void* bias_ptr = bias.has_value() && bias->defined() ? bias->data_ptr() : nullptr;
    check_rc(b2_w4a16_linear_flags(x.data_ptr(), m > 1 ? x.stride(0) : k, image.data_ptr(), bias_ptr, y.data_ptr(), n, m, n, k,
                                   ws.data_ptr(), ws.numel(), stream, int(route), int(flags)));
    return y;
}

enum class Rule { Any, Small, Gemv, Naive };

template <Rule R>
at::Tensor legacy_op(const at::Tensor& x, const at::Tensor& packed, const at::Tensor& scales, const at::Tensor& zeros,
                     int64_t group_size) {
    check_w4a16(x, packed, scales, zeros, group_size);
    if (R == Rule::Any) TORCH_CHECK(group_size == 64, "W4A16 Tensor Core backend requires group_size=64");
    if (R == Rule::Small) TORCH_CHECK(group_size == 64 && x.size(0) <= 8, "W4A16 small requires group_size=64 and M<=8");
    if (R == Rule::Gemv) TORCH_CHECK(x.size(0) == 1, "w4a16_gemv expects x=[1,K]");
    if (R == Rule::Gemv || R == Rule::Naive) TORCH_CHECK(group_size == 64, "this W4A16 engine requires group_size=64");
    c10::cuda::CUDAGuard guard(x.device());
    return run_image(x, image_for(packed, scales, zeros, x.size(1)), packed.size(0), x.size(1), c10::nullopt, B2_ROUTE_AUTO);
}

// x [M, K] FP16 with unit inner stride, image = device-native weight image, bias = FP16 [N] or None,
// flags = layer flags of the C ABI (B2_FLAG_FP16_STEPS).
at::Tensor linear_image(const at::Tensor& x, const at::Tensor& image, int64_t n, int64_t k, const c10::optional<at::Tensor>& bias,
                        int64_t route, int64_t flags) {
    TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kHalf && x.dim() == 2 && x.size(1) == k && x.stride(1) == 1 &&
                    (x.size(0) <= 1 || x.stride(0) >= k), "x must be a CUDA FP16 [M, K] tensor with unit inner stride");
    TORCH_CHECK(image.is_cuda() && image.scalar_type() == at::kByte && image.device() == x.device() &&
                    image.numel() == b2_w4a16_native_bytes(n, k), "not a native image of an [N, K] layer on x's device");
    if (bias.has_value() && bias->defined())
        TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kHalf && bias->numel() == n && bias->is_contiguous(),
                    "bias must be a contiguous CUDA FP16 [N] tensor");
    return run_image(x, image, n, k, bias, route, flags);
}

int64_t status_all() {
    std::vector<at::Tensor> buffers;
    {
        std::lock_guard<std::mutex> lock(g_mutex);
        for (auto& kv : pool().live) buffers.push_back(kv.second);
        for (auto& t : pool().retired) buffers.push_back(t);
    }
    unsigned all = 0;
    for (auto& t : buffers) {
        c10::cuda::CUDAGuard guard(t.device());
        unsigned word = 0;
        check_rc(b2_w4a16_status(t.data_ptr(), at::cuda::getCurrentCUDAStream().stream(), &word));
        all |= word;
    }
    return int64_t(all);
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(dandan_ops, m) {
    m.def("w4a16_contract_version() -> int", []() -> int64_t { return b2_w4a16_contract_version(); });
    m.def("w4a16_gemm(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor");
    m.def("w4a16_gemv(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor");
    m.def("w4a16_tensorcore(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor");
    m.def("w4a16_small(Tensor x, Tensor packed_w, Tensor scales, Tensor zeros, int group_size) -> Tensor");
    m.def("w4a16_linear_image(Tensor x, Tensor image, int n, int k, Tensor? bias, int route, int flags) -> Tensor");
    m.def("w4a16_workspace_status() -> int", &status_all);
}

TORCH_LIBRARY_IMPL(dandan_ops, CUDA, m) {
    m.impl("w4a16_gemm", &legacy_op<Rule::Naive>);
    m.impl("w4a16_gemv", &legacy_op<Rule::Gemv>);
    m.impl("w4a16_tensorcore", &legacy_op<Rule::Any>);
    m.impl("w4a16_small", &legacy_op<Rule::Small>);
    m.impl("w4a16_linear_image", &linear_image);
}
