// pybind11 module `xstar_cpp`: the Tensor bridge functions the reference's tests use
// (reference bindings/python_bindings.cpp:60-135, 389-410: from_numpy_raw / to_numpy_raw / to_cuda / to_cpu /
// cuda_free_bytes, DType, Device, Tensor) plus the MoE op.  Raw bytes cross the boundary; numpy dtypes carry
// no meaning beyond their item size (bf16 travels as uint16, e4m3 / packed e2m1 / e8m0 as uint8).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "cuda/cuda_allocator.h"
#include "ops/moe.h"
#include "ops/moe_ep.h"
#include "parallel/ep_group.h"
#include "parallel/ep_scheduler.h"
#include "tensor.h"
#include "weight_io.h"

namespace py = pybind11;

namespace {

Tensor from_numpy_raw(py::array array, std::vector<std::int64_t> shape, DType dtype)
{
    if (static_cast<std::size_t>(array.itemsize()) != dtype_size(dtype))
        throw std::runtime_error("itemsize mismatch: array itemsize != dtype size");
    std::int64_t n = 1;
    for (auto s : shape)
        n *= s;
    if (array.size() != n)
        throw std::runtime_error("byte count mismatch");
    if (!(array.flags() & py::array::c_style))
        throw std::runtime_error("array must be C-contiguous");
    Tensor t(std::move(shape), dtype, Device::CPU);
    std::memcpy(t.data(), array.data(), t.nbytes());
    return t;
}

py::array to_numpy_raw(const Tensor &t)
{
    if (t.device() != Device::CPU)
        throw std::runtime_error("to_numpy_raw: tensor is not on the CPU");
    py::array_t<std::uint8_t> out(static_cast<py::ssize_t>(t.nbytes()));
    std::memcpy(out.mutable_data(), t.data(), t.nbytes());
    return out;
}

const Tensor *opt(py::object o)
{
    return o.is_none() ? nullptr : &o.cast<const Tensor &>();
}

MoEWeights weights_of(const Tensor &router_weight, const Tensor &gate_up_weight, const Tensor &down_weight, py::object router_bias,
                      py::object gate_up_scale, py::object down_scale, py::object shared_gate_up_weight, py::object shared_down_weight,
                      py::object shared_gate_up_scale, py::object shared_down_scale)
{
    MoEWeights w;
    w.router_weight = &router_weight;
    w.router_bias = opt(router_bias);
    w.gate_up_weight = &gate_up_weight;
    w.gate_up_scale = opt(gate_up_scale);
    w.down_weight = &down_weight;
    w.down_scale = opt(down_scale);
    w.shared_gate_up_weight = opt(shared_gate_up_weight);
    w.shared_down_weight = opt(shared_down_weight);
    w.shared_gate_up_scale = opt(shared_gate_up_scale);
    w.shared_down_scale = opt(shared_down_scale);
    return w;
}

Tensor moe_py(const Tensor &x, const Tensor &router_weight, const Tensor &gate_up_weight, const Tensor &down_weight, std::int64_t top_k,
              py::object router_bias, py::object gate_up_scale, py::object down_scale, py::object shared_gate_up_weight,
              py::object shared_down_weight, py::object shared_gate_up_scale, py::object shared_down_scale)
{
    MoEWeights w = weights_of(router_weight, gate_up_weight, down_weight, router_bias, gate_up_scale, down_scale, shared_gate_up_weight,
                              shared_down_weight, shared_gate_up_scale, shared_down_scale);
    MoEConfig cfg;
    cfg.top_k = top_k;
    py::gil_scoped_release nogil; // the device work does not touch Python state
    return moe(x, w, cfg);
}

Tensor moe_block_py(const Tensor &x, const Tensor &norm_weight, float eps, const Tensor &router_weight, const Tensor &gate_up_weight,
                    const Tensor &down_weight, std::int64_t top_k, py::object router_bias, py::object gate_up_scale, py::object down_scale,
                    py::object shared_gate_up_weight, py::object shared_down_weight, py::object shared_gate_up_scale,
                    py::object shared_down_scale)
{
    MoEWeights w = weights_of(router_weight, gate_up_weight, down_weight, router_bias, gate_up_scale, down_scale, shared_gate_up_weight,
                              shared_down_weight, shared_gate_up_scale, shared_down_scale);
    MoEConfig cfg;
    cfg.top_k = top_k;
    py::gil_scoped_release nogil;
    return moe_block(x, norm_weight, eps, w, cfg);
}

EpShape ep_shape(std::int64_t max_tokens, std::int64_t hidden, std::int64_t experts, std::int64_t top_k, std::int64_t intermediate,
                 DType expert_dtype, bool shared)
{
    EpShape s;
    s.max_tokens = max_tokens;
    s.hidden = hidden;
    s.experts = experts;
    s.top_k = top_k;
    s.intermediate = intermediate;
    s.expert_dtype = expert_dtype;
    s.shared = shared;
    return s;
}

py::dict moe_route_py(const Tensor &x, const Tensor &router_weight, std::int64_t top_k, py::object router_bias)
{
    MoEConfig cfg;
    cfg.top_k = top_k;
    MoERouting r = moe_route(x, router_weight, opt(router_bias), cfg);
    const py::ssize_t T = x.dim(-1) ? x.numel() / x.dim(-1) : 0, K = top_k;
    auto ivec = [](const std::vector<std::int32_t> &v, std::vector<py::ssize_t> shape) {
        py::array_t<std::int32_t> a(shape);
        std::memcpy(a.mutable_data(), v.data(), v.size() * 4);
        return a;
    };
    py::array_t<float> w({T, K});
    std::memcpy(w.mutable_data(), r.topk_weights.data(), r.topk_weights.size() * 4);
    py::dict d;
    d["topk_ids"] = ivec(r.topk_ids, {T, K});
    d["topk_w"] = w;
    d["counts"] = ivec(r.counts, {(py::ssize_t)r.counts.size()});
    d["offsets"] = ivec(r.offsets, {(py::ssize_t)r.offsets.size()});
    d["perm"] = ivec(r.perm, {(py::ssize_t)r.perm.size()});
    d["inv"] = ivec(r.inv, {(py::ssize_t)r.inv.size()});
    return d;
}

} // namespace

PYBIND11_MODULE(xstar_cpp, m)
{
    m.doc() = "Xstar MoE layer for B200: Tensor bridge + moe op";

    py::enum_<DType>(m, "DType")
        .value("Float32", DType::Float32)
        .value("BFloat16", DType::BFloat16)
        .value("Float8E4M3", DType::Float8E4M3)
        .value("Float4E2M1x2", DType::Float4E2M1x2)
        .value("UE8M0", DType::UE8M0)
        .value("Int32", DType::Int32)
        .value("UInt8", DType::UInt8)
        .export_values();
    py::enum_<Device>(m, "Device").value("CPU", Device::CPU).value("CUDA", Device::CUDA).export_values();

    py::class_<Tensor>(m, "Tensor")
        .def(py::init<std::vector<std::int64_t>, DType, Device>(), py::arg("shape"), py::arg("dtype"), py::arg("device") = Device::CPU)
        .def("numel", &Tensor::numel)
        .def("nbytes", &Tensor::nbytes)
        .def("shape", &Tensor::shape)
        .def("dtype", &Tensor::dtype)
        .def("device", &Tensor::device);

    m.def("from_numpy_raw", &from_numpy_raw, py::arg("array"), py::arg("shape"), py::arg("dtype"));
    m.def("to_numpy_raw", &to_numpy_raw, py::arg("tensor"));
    // borrowed view of device memory another owner keeps alive (a framework's tensor): no copy, no ownership
    m.def(
        "from_device_ptr",
        [](std::uintptr_t ptr, std::vector<std::int64_t> shape, DType dtype) {
            return Tensor(reinterpret_cast<const void *>(ptr), std::move(shape), dtype, Device::CUDA);
        },
        py::arg("ptr"), py::arg("shape"), py::arg("dtype"));
    m.def("to_cuda", &to_cuda, py::arg("tensor"));
    m.def("to_cpu", &to_cpu, py::arg("tensor"));
    m.def("cuda_free_bytes", &cuda_free_bytes);
    m.def("workspace_cached_bytes", [] { return WorkspacePool::instance().cached_bytes(); });
    m.def("workspace_trim", [] {
        WorkspacePool::instance().trim();
        cuda_trim_cached();
    });
    m.def("result_cache_bytes", &cuda_cached_result_bytes);
    py::class_<MoEScratch>(m, "MoEScratch").def(py::init<>()).def("bytes", &MoEScratch::bytes);
    m.def(
        "moe_into",
        [](const Tensor &x, Tensor &out, MoEScratch &scratch, std::uintptr_t stream, const Tensor &router_weight, const Tensor &gate_up_weight,
           const Tensor &down_weight, std::int64_t top_k, py::object router_bias, py::object gate_up_scale, py::object down_scale,
           py::object shared_gate_up_weight, py::object shared_down_weight, py::object shared_gate_up_scale, py::object shared_down_scale) {
            MoEWeights w = weights_of(router_weight, gate_up_weight, down_weight, router_bias, gate_up_scale, down_scale, shared_gate_up_weight,
                                      shared_down_weight, shared_gate_up_scale, shared_down_scale);
            MoEConfig cfg;
            cfg.top_k = top_k;
            py::gil_scoped_release nogil;
            moe_into(x, w, cfg, out, scratch, reinterpret_cast<void *>(stream));
        },
        py::arg("x"), py::arg("out"), py::arg("scratch"), py::arg("stream"), py::arg("router_weight"), py::arg("gate_up_weight"),
        py::arg("down_weight"), py::arg("top_k"), py::arg("router_bias") = py::none(), py::arg("gate_up_scale") = py::none(),
        py::arg("down_scale") = py::none(), py::arg("shared_gate_up_weight") = py::none(), py::arg("shared_down_weight") = py::none(),
        py::arg("shared_gate_up_scale") = py::none(), py::arg("shared_down_scale") = py::none());
    m.def("moe_check", [](MoEScratch &s, std::uintptr_t stream) { moe_check(s, reinterpret_cast<void *>(stream)); }, py::arg("scratch"),
          py::arg("stream") = 0, py::call_guard<py::gil_scoped_release>());

    m.def("moe", &moe_py, py::arg("x"), py::arg("router_weight"), py::arg("gate_up_weight"), py::arg("down_weight"), py::arg("top_k"),
          py::arg("router_bias") = py::none(), py::arg("gate_up_scale") = py::none(), py::arg("down_scale") = py::none(),
          py::arg("shared_gate_up_weight") = py::none(), py::arg("shared_down_weight") = py::none(),
          py::arg("shared_gate_up_scale") = py::none(), py::arg("shared_down_scale") = py::none());
    m.def("moe_block", &moe_block_py, py::arg("x"), py::arg("norm_weight"), py::arg("eps"), py::arg("router_weight"),
          py::arg("gate_up_weight"), py::arg("down_weight"), py::arg("top_k"), py::arg("router_bias") = py::none(),
          py::arg("gate_up_scale") = py::none(), py::arg("down_scale") = py::none(), py::arg("shared_gate_up_weight") = py::none(),
          py::arg("shared_down_weight") = py::none(), py::arg("shared_gate_up_scale") = py::none(),
          py::arg("shared_down_scale") = py::none());
    // checkpoint IO (same names as the reference's module: MMapFile, parse_safetensors_header, make_weight_view)
    py::class_<MMapFile>(m, "MMapFile").def(py::init<const std::string &>(), py::arg("path")).def("size", &MMapFile::size);
    py::class_<TensorMeta>(m, "TensorMeta")
        .def_readonly("offset", &TensorMeta::offset)
        .def_readonly("shape", &TensorMeta::shape)
        .def_readonly("dtype", &TensorMeta::dtype);
    m.def("parse_safetensors_header", &parse_safetensors_header, py::arg("file"));
    m.def("make_weight_view", &make_weight_view, py::arg("file"), py::arg("offset"), py::arg("shape"), py::arg("dtype"),
          py::keep_alive<0, 1>()); // the view borrows the mapping
    py::class_<MoeLayerWeights>(m, "MoeLayerWeights")
        .def_readonly("num_experts", &MoeLayerWeights::num_experts)
        .def_readonly("first_expert", &MoeLayerWeights::first_expert)
        .def_readonly("expert_count", &MoeLayerWeights::expert_count)
        .def_readonly("hidden", &MoeLayerWeights::hidden)
        .def_readonly("intermediate", &MoeLayerWeights::intermediate)
        .def_property_readonly("router_weight", [](const MoeLayerWeights &w) { return &w.router_weight; }, py::return_value_policy::reference_internal)
        .def_property_readonly("gate_up_weight", [](const MoeLayerWeights &w) { return &w.gate_up_weight; }, py::return_value_policy::reference_internal)
        .def_property_readonly("down_weight", [](const MoeLayerWeights &w) { return &w.down_weight; }, py::return_value_policy::reference_internal)
        .def("optional",
             [](const MoeLayerWeights &w, const std::string &name) -> const Tensor * {
                 const std::optional<Tensor> *o = name == "router_bias"             ? &w.router_bias
                                                  : name == "gate_up_scale"         ? &w.gate_up_scale
                                                  : name == "down_scale"            ? &w.down_scale
                                                  : name == "shared_gate_up_weight" ? &w.shared_gate_up_weight
                                                  : name == "shared_down_weight"    ? &w.shared_down_weight
                                                  : name == "shared_gate_up_scale"  ? &w.shared_gate_up_scale
                                                  : name == "shared_down_scale"     ? &w.shared_down_scale
                                                                                    : nullptr;
                 if (!o)
                     throw std::runtime_error("unknown tensor name");
                 return o->has_value() ? &o->value() : nullptr;
             },
             py::arg("name"), py::return_value_policy::reference_internal);
    m.def("load_moe_layer", &load_moe_layer, py::arg("file"), py::arg("meta"), py::arg("prefix"), py::arg("num_experts"),
          py::arg("first_expert"), py::arg("expert_count"), py::arg("device") = Device::CPU, py::call_guard<py::gil_scoped_release>());
    m.def("set_device", &cuda_set_device, py::arg("device"));
    m.def("current_device", &cuda_current_device);
    m.def("ep_unique_id", [] {
        const EpUniqueId id = ep_unique_id();
        return py::bytes(reinterpret_cast<const char *>(id.data()), id.size());
    });
    m.def("ep_capacity_rows", &ep_capacity_rows, py::arg("max_tokens"), py::arg("top_k"), py::arg("world"), py::arg("capacity_factor"));
    py::register_exception<EpError>(m, "EpError", PyExc_RuntimeError);
    py::class_<EpGroup, std::shared_ptr<EpGroup>>(m, "EpGroup")
        .def(py::init([](int world, int timeout_ms) { return std::make_shared<EpGroup>(world, std::chrono::milliseconds(timeout_ms)); }),
             py::arg("world"), py::arg("timeout_ms") = 30000)
        .def("arrive", &EpGroup::arrive, py::arg("rank"), py::arg("signature"), py::call_guard<py::gil_scoped_release>())
        .def("leave", &EpGroup::leave, py::arg("rank"))
        .def("broken", &EpGroup::broken)
        .def("world", &EpGroup::world);
    py::class_<EpContext>(m, "EpContext")
        .def(py::init([](std::shared_ptr<EpGroup> group, py::bytes id, int rank, int world, int device, std::int64_t max_tokens,
                         std::int64_t hidden, std::int64_t experts, std::int64_t top_k, std::int64_t intermediate, DType expert_dtype,
                         bool shared, double capacity_factor, bool fused_return, bool signal_barriers) {
                 const std::string raw = id;
                 if (raw.size() != 128)
                     throw std::runtime_error("unique id must be 128 bytes");
                 EpUniqueId u;
                 std::memcpy(u.data(), raw.data(), 128);
                 EpOptions o;
                 o.capacity_factor = capacity_factor;
                 o.fused_return = fused_return;
                 o.signal_barriers = signal_barriers;
                 const EpShape s = ep_shape(max_tokens, hidden, experts, top_k, intermediate, expert_dtype, shared);
                 py::gil_scoped_release nogil; // collective: the other ranks' threads must be able to run
                 return std::make_unique<EpContext>(std::move(group), u, rank, world, device, s, o);
             }),
             py::arg("group"), py::arg("unique_id"), py::arg("rank"), py::arg("world"), py::arg("device"), py::arg("max_tokens"),
             py::arg("hidden"), py::arg("experts"), py::arg("top_k"), py::arg("intermediate"), py::arg("expert_dtype"), py::arg("shared"),
             py::arg("capacity_factor") = 0.0, py::arg("fused_return") = true, py::arg("signal_barriers") = true)
        .def("rank", &EpContext::rank)
        .def("fused_return", &EpContext::fused_return)
        .def("signal_barriers", &EpContext::signal_barriers)
        .def("world", &EpContext::world)
        .def("capacity_rows", &EpContext::capacity_rows)
        .def("abandon", &EpContext::abandon)
        .def("check", [](EpContext &c, std::uintptr_t stream) { c.check(reinterpret_cast<void *>(stream)); }, py::arg("stream") = 0,
             py::call_guard<py::gil_scoped_release>())
        .def(
            "moe",
            [](EpContext &c, const Tensor &x, const Tensor &router_weight, const Tensor &gate_up_weight, const Tensor &down_weight,
               std::int64_t top_k, py::object router_bias, py::object gate_up_scale, py::object down_scale, py::object shared_gate_up_weight,
               py::object shared_down_weight, py::object shared_gate_up_scale, py::object shared_down_scale) {
                MoEWeights w = weights_of(router_weight, gate_up_weight, down_weight, router_bias, gate_up_scale, down_scale,
                                          shared_gate_up_weight, shared_down_weight, shared_gate_up_scale, shared_down_scale);
                MoEConfig cfg;
                cfg.top_k = top_k;
                py::gil_scoped_release nogil;
                return moe(x, w, cfg, &c);
            },
            py::arg("x"), py::arg("router_weight"), py::arg("gate_up_weight"), py::arg("down_weight"), py::arg("top_k"),
            py::arg("router_bias") = py::none(), py::arg("gate_up_scale") = py::none(), py::arg("down_scale") = py::none(),
            py::arg("shared_gate_up_weight") = py::none(), py::arg("shared_down_weight") = py::none(),
            py::arg("shared_gate_up_scale") = py::none(), py::arg("shared_down_scale") = py::none())
        .def(
            "moe_into",
            [](EpContext &c, const Tensor &x, Tensor &out, std::uintptr_t stream, const Tensor &router_weight, const Tensor &gate_up_weight,
               const Tensor &down_weight, std::int64_t top_k, py::object router_bias, py::object gate_up_scale, py::object down_scale,
               py::object shared_gate_up_weight, py::object shared_down_weight, py::object shared_gate_up_scale, py::object shared_down_scale) {
                MoEWeights w = weights_of(router_weight, gate_up_weight, down_weight, router_bias, gate_up_scale, down_scale,
                                          shared_gate_up_weight, shared_down_weight, shared_gate_up_scale, shared_down_scale);
                MoEConfig cfg;
                cfg.top_k = top_k;
                py::gil_scoped_release nogil;
                c.forward_into(x, w, cfg, out, reinterpret_cast<void *>(stream));
            },
            py::arg("x"), py::arg("out"), py::arg("stream"), py::arg("router_weight"), py::arg("gate_up_weight"), py::arg("down_weight"),
            py::arg("top_k"), py::arg("router_bias") = py::none(), py::arg("gate_up_scale") = py::none(), py::arg("down_scale") = py::none(),
            py::arg("shared_gate_up_weight") = py::none(), py::arg("shared_down_weight") = py::none(),
            py::arg("shared_gate_up_scale") = py::none(), py::arg("shared_down_scale") = py::none());
    m.def(
        "ep_balance_batch",
        [](const std::vector<std::int64_t> &cu_seqlens, int ranks, std::int64_t max_tokens_per_rank) {
            const EpBatchPlan p = ep_balance_batch(cu_seqlens, ranks, max_tokens_per_rank);
            py::dict d;
            d["sequences_of_rank"] = p.sequences_of_rank;
            d["tokens_of_rank"] = p.tokens_of_rank;
            d["rank_of_sequence"] = p.rank_of_sequence;
            d["max_tokens"] = p.max_tokens();
            d["imbalance"] = p.imbalance();
            return d;
        },
        py::arg("cu_seqlens"), py::arg("ranks"), py::arg("max_tokens_per_rank") = 0);
    py::class_<EpWorkerPool>(m, "EpWorkerPool")
        .def(py::init([](int world, std::vector<int> devices, std::int64_t max_tokens, std::int64_t hidden, std::int64_t experts,
                         std::int64_t top_k, std::int64_t intermediate, DType expert_dtype, bool shared, double capacity_factor, int timeout_ms) {
                 EpOptions o;
                 o.capacity_factor = capacity_factor;
                 const EpShape s = ep_shape(max_tokens, hidden, experts, top_k, intermediate, expert_dtype, shared);
                 py::gil_scoped_release nogil;
                 return std::make_unique<EpWorkerPool>(world, std::move(devices), s, o, std::chrono::milliseconds(timeout_ms));
             }),
             py::arg("world"), py::arg("devices"), py::arg("max_tokens"), py::arg("hidden"), py::arg("experts"), py::arg("top_k"),
             py::arg("intermediate"), py::arg("expert_dtype"), py::arg("shared"), py::arg("capacity_factor") = 0.0, py::arg("timeout_ms") = 30000)
        .def("world", &EpWorkerPool::world)
        // per-rank lists: x[r], router_weight[r], gate_up_weight[r], down_weight[r]; the optional lists hold one tensor per rank
        .def(
            "run",
            [](EpWorkerPool &pool, py::list x, py::list router_weight, py::list gate_up_weight, py::list down_weight, std::int64_t top_k,
               py::object router_bias, py::object gate_up_scale, py::object down_scale, py::object shared_gate_up_weight,
               py::object shared_down_weight, py::object shared_gate_up_scale, py::object shared_down_scale) {
                const int R = pool.world();
                auto at = [&](py::object lst, int r) -> py::object {
                    if (lst.is_none())
                        return py::none();
                    py::list l = lst.cast<py::list>();
                    if (static_cast<int>(l.size()) != R)
                        throw std::runtime_error("bad rank count");
                    return l[r];
                };
                std::vector<const Tensor *> xs(R);
                std::vector<MoEWeights> ws(R);
                for (int r = 0; r < R; r++) {
                    xs[r] = &at(x, r).cast<const Tensor &>();
                    ws[r] = weights_of(at(router_weight, r).cast<const Tensor &>(), at(gate_up_weight, r).cast<const Tensor &>(),
                                       at(down_weight, r).cast<const Tensor &>(), at(router_bias, r), at(gate_up_scale, r), at(down_scale, r),
                                       at(shared_gate_up_weight, r), at(shared_down_weight, r), at(shared_gate_up_scale, r),
                                       at(shared_down_scale, r));
                }
                MoEConfig cfg;
                cfg.top_k = top_k;
                std::vector<Tensor> out;
                {
                    py::gil_scoped_release nogil;
                    out = pool.run(xs, ws, cfg);
                }
                py::list res;
                for (auto &t : out)
                    res.append(py::cast(std::move(t)));
                return res;
            },
            py::arg("x"), py::arg("router_weight"), py::arg("gate_up_weight"), py::arg("down_weight"), py::arg("top_k"),
            py::arg("router_bias") = py::none(), py::arg("gate_up_scale") = py::none(), py::arg("down_scale") = py::none(),
            py::arg("shared_gate_up_weight") = py::none(), py::arg("shared_down_weight") = py::none(),
            py::arg("shared_gate_up_scale") = py::none(), py::arg("shared_down_scale") = py::none());
    m.def("moe_route", &moe_route_py, py::arg("x"), py::arg("router_weight"), py::arg("top_k"), py::arg("router_bias") = py::none());
}
