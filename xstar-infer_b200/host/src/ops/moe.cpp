#include "ops/moe.h"

#include <stdexcept>
#include <string>

#include "cuda/cuda_allocator.h"
#include "ops/moe_checked.h"
#include "xs_moe.h"

namespace moe_detail {

void raise_if(int rc)
{
    if (rc != 0)
        throw std::runtime_error(std::string(xs_moe_last_error()));
}

int format_of(const Tensor &w)
{
    switch (w.dtype()) {
    case DType::BFloat16: return XS_MOE_BF16;
    case DType::Float8E4M3: return XS_MOE_FP8_BLOCK128;
    case DType::Float4E2M1x2: return XS_MOE_FP4_MX32;
    default: throw std::runtime_error("unsupported dtype");
    }
}

// validation in the order the reference's ops use: dtype, rank, shape, device
Checked validate(const Tensor &x, const MoEWeights &m, const MoEConfig &config, bool need_experts, std::int64_t local_experts)
{
    if (!m.router_weight || (need_experts && (!m.gate_up_weight || !m.down_weight)))
        throw std::runtime_error("missing weight");
    const Tensor &rw = *m.router_weight;
    if (x.dtype() != DType::BFloat16 || rw.dtype() != DType::BFloat16)
        throw std::runtime_error("dtype mismatch");
    if (m.router_bias && m.router_bias->dtype() != DType::Float32)
        throw std::runtime_error("dtype mismatch");
    if (x.rank() < 1 || rw.rank() != 2 || (m.router_bias && m.router_bias->rank() != 1))
        throw std::runtime_error("rank mismatch");
    const std::int64_t H = x.dim(-1), E = rw.dim(0);
    if (rw.dim(1) != H || (m.router_bias && m.router_bias->dim(0) != E))
        throw std::runtime_error("shape mismatch");
    if (config.top_k < 1 || config.top_k > E)
        throw std::runtime_error("top_k out of range");
    if (x.device() != rw.device() || (m.router_bias && m.router_bias->device() != x.device()))
        throw std::runtime_error("device mismatch");

    Checked c;
    c.cfg.num_tokens = static_cast<int32_t>(H ? x.numel() / H : 0);
    c.cfg.hidden = static_cast<int32_t>(H);
    c.cfg.num_experts = static_cast<int32_t>(E);
    c.cfg.top_k = static_cast<int32_t>(config.top_k);
    c.cfg.local_expert_count = static_cast<int32_t>(E);
    c.cfg.intermediate = 128; // placeholder for routing-only calls
    c.w.router_w_dev = rw.data();
    c.w.router_bias_dev = m.router_bias ? m.router_bias->data<float>() : nullptr;
    if (!need_experts)
        return c;

    const Tensor &gu = *m.gate_up_weight, &dw = *m.down_weight;
    if (gu.dtype() != dw.dtype())
        throw std::runtime_error("dtype mismatch");
    const int fmt = format_of(gu);
    if (gu.rank() != 3 || dw.rank() != 3)
        throw std::runtime_error("rank mismatch");
    const std::int64_t held = local_experts >= 0 ? local_experts : E; // expert-parallel ranks hold a slice of the experts
    if (gu.dim(0) != held || dw.dim(0) != held)
        throw std::runtime_error("expert count mismatch");
    if (gu.dim(1) % 2 != 0)
        throw std::runtime_error("gate_up out must be even");
    const std::int64_t I = gu.dim(1) / 2;
    const std::int64_t kdiv = (fmt == XS_MOE_FP4_MX32) ? 2 : 1; // packed nibbles: last dim counts bytes
    if (gu.dim(2) * kdiv != H || dw.dim(1) != H || dw.dim(2) * kdiv != I)
        throw std::runtime_error("shape mismatch");
    if (gu.device() != x.device() || dw.device() != x.device())
        throw std::runtime_error("device mismatch");
    if (fmt != XS_MOE_BF16) {
        if (!m.gate_up_scale || !m.down_scale)
            throw std::runtime_error("missing scale");
        if (m.gate_up_scale->device() != x.device() || m.down_scale->device() != x.device())
            throw std::runtime_error("device mismatch");
        if (fmt == XS_MOE_FP8_BLOCK128) {
            if (m.gate_up_scale->dtype() != DType::Float32 || m.down_scale->dtype() != DType::Float32)
                throw std::runtime_error("dtype mismatch");
            if (m.gate_up_scale->numel() != held * (2 * I / 128) * (H / 128) || m.down_scale->numel() != held * (H / 128) * (I / 128))
                throw std::runtime_error("shape mismatch");
        } else {
            if (m.gate_up_scale->dtype() != DType::UE8M0 || m.down_scale->dtype() != DType::UE8M0)
                throw std::runtime_error("dtype mismatch");
            if (m.gate_up_scale->numel() != held * 2 * I * (H / 32) || m.down_scale->numel() != held * H * (I / 32))
                throw std::runtime_error("shape mismatch");
        }
    }
    c.cfg.intermediate = static_cast<int32_t>(I);
    c.cfg.routed_format = fmt;
    c.cfg.shared_format = fmt;
    c.w.gate_up_w_dev = gu.data();
    c.w.down_w_dev = dw.data();
    c.w.gate_up_scale_dev = m.gate_up_scale ? m.gate_up_scale->data() : nullptr;
    c.w.down_scale_dev = m.down_scale ? m.down_scale->data() : nullptr;

    if ((m.shared_gate_up_weight != nullptr) != (m.shared_down_weight != nullptr))
        throw std::runtime_error("missing weight");
    if (m.shared_gate_up_weight) {
        const Tensor &sg = *m.shared_gate_up_weight, &sd = *m.shared_down_weight;
        if (sg.dtype() != sd.dtype())
            throw std::runtime_error("dtype mismatch");
        const int sfmt = format_of(sg);
        if (sfmt == XS_MOE_FP4_MX32)
            throw std::runtime_error("unsupported dtype");
        if (sg.rank() != 2 || sd.rank() != 2)
            throw std::runtime_error("rank mismatch");
        if (sg.dim(0) != 2 * I || sg.dim(1) != H || sd.dim(0) != H || sd.dim(1) != I)
            throw std::runtime_error("shape mismatch");
        if (sg.device() != x.device() || sd.device() != x.device())
            throw std::runtime_error("device mismatch");
        if (sfmt == XS_MOE_FP8_BLOCK128) {
            if (!m.shared_gate_up_scale || !m.shared_down_scale)
                throw std::runtime_error("missing scale");
            if (m.shared_gate_up_scale->dtype() != DType::Float32 || m.shared_down_scale->dtype() != DType::Float32)
                throw std::runtime_error("dtype mismatch");
            c.w.shared_gate_up_scale_dev = m.shared_gate_up_scale->data();
            c.w.shared_down_scale_dev = m.shared_down_scale->data();
        }
        c.cfg.num_shared = 1;
        c.cfg.shared_format = sfmt;
        c.w.shared_gate_up_w_dev = sg.data();
        c.w.shared_down_w_dev = sd.data();
    }
    return c;
}

} // namespace moe_detail

using moe_detail::Checked;
using moe_detail::raise_if;

MoEScratch::~MoEScratch()
{
    if (ptr_) {
        WorkspacePool::Lease l;
        l.ptr = ptr_;
        l.bytes = bytes_;
        l.device = device_;
        WorkspacePool::instance().release(l);
    }
}

void MoEScratch::reserve(std::size_t bytes)
{
    if (bytes <= bytes_ && ptr_)
        return;
    if (ptr_) {
        raise_if(xs_moe_stream_synchronize(nullptr)); // legacy default stream: waits for every blocking stream of the device
        WorkspacePool::Lease old;
        old.ptr = ptr_;
        old.bytes = bytes_;
        old.device = device_;
        WorkspacePool::instance().release(old);
        ptr_ = nullptr;
        bytes_ = 0;
    }
    WorkspacePool::Lease l = WorkspacePool::instance().acquire(bytes);
    ptr_ = l.ptr;
    bytes_ = l.bytes;
    device_ = l.device;
}

namespace {
void check_out(const Tensor &x, const Tensor &out)
{
    if (out.dtype() != DType::BFloat16)
        throw std::runtime_error("dtype mismatch");
    if (out.numel() != x.numel())
        throw std::runtime_error("shape mismatch");
    if (out.device() != Device::CUDA || x.device() != Device::CUDA)
        throw std::runtime_error("unsupported device");
}
} // namespace

void moe_into(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, Tensor &out, MoEScratch &scratch, void *stream)
{
    Checked c = moe_detail::validate(x, weights, config, true);
    check_out(x, out);
    std::size_t need = 0;
    raise_if(xs_moe_workspace_bytes(&c.cfg, &need));
    scratch.reserve(need);
    raise_if(xs_moe_forward(&c.cfg, &c.w, x.data(), out.data(), scratch.data(), scratch.bytes(), stream));
}

void moe_block_into(const Tensor &x, const Tensor &norm_weight, float eps, const MoEWeights &weights, const MoEConfig &config, Tensor &out,
                    MoEScratch &scratch, void *stream)
{
    if (norm_weight.dtype() != DType::BFloat16)
        throw std::runtime_error("dtype mismatch");
    if (norm_weight.rank() != 1)
        throw std::runtime_error("rank mismatch");
    Checked c = moe_detail::validate(x, weights, config, true);
    if (norm_weight.dim(0) != x.dim(-1))
        throw std::runtime_error("shape mismatch");
    if (norm_weight.device() != x.device())
        throw std::runtime_error("device mismatch");
    check_out(x, out);
    std::size_t need = 0;
    raise_if(xs_moe_block_workspace_bytes(&c.cfg, &need));
    scratch.reserve(need);
    raise_if(xs_moe_block_forward(&c.cfg, &c.w, x.data(), norm_weight.data(), eps, out.data(), scratch.data(), scratch.bytes(), stream));
}

void moe_check(MoEScratch &scratch, void *stream)
{
    if (scratch.data())
        raise_if(xs_moe_check_flags(scratch.data(), stream));
    else
        raise_if(xs_moe_stream_synchronize(stream));
}

Tensor moe(const Tensor &x, const MoEWeights &weights, const MoEConfig &config)
{
    Checked c = moe_detail::validate(x, weights, config, true);
    if (x.device() != Device::CUDA)
        throw std::runtime_error("unsupported device");
    std::size_t need = 0;
    raise_if(xs_moe_workspace_bytes(&c.cfg, &need));
    Tensor out = Tensor::result(x.shape(), DType::BFloat16);
    Workspace ws(need);
    // explicit stream semantics of the engine: default stream, and "returns => finished"
    // (reference xstar_cpp/src/ops/mlp.cu:188-189), with ONE synchronisation at op exit
    raise_if(xs_moe_forward(&c.cfg, &c.w, x.data(), out.data(), ws.data(), ws.bytes(), nullptr));
    raise_if(xs_moe_check_flags(ws.data(), nullptr));
    return out;
}

Tensor moe_block(const Tensor &x, const Tensor &norm_weight, float eps, const MoEWeights &weights, const MoEConfig &config)
{
    if (norm_weight.dtype() != DType::BFloat16)
        throw std::runtime_error("dtype mismatch");
    if (norm_weight.rank() != 1)
        throw std::runtime_error("rank mismatch");
    Checked c = moe_detail::validate(x, weights, config, true);
    if (norm_weight.dim(0) != x.dim(-1))
        throw std::runtime_error("shape mismatch");
    if (norm_weight.device() != x.device())
        throw std::runtime_error("device mismatch");
    if (x.device() != Device::CUDA)
        throw std::runtime_error("unsupported device");
    std::size_t need = 0;
    raise_if(xs_moe_block_workspace_bytes(&c.cfg, &need));
    Tensor out = Tensor::result(x.shape(), DType::BFloat16);
    Workspace ws(need);
    raise_if(xs_moe_block_forward(&c.cfg, &c.w, x.data(), norm_weight.data(), eps, out.data(), ws.data(), ws.bytes(), nullptr));
    raise_if(xs_moe_check_flags(ws.data(), nullptr));
    return out;
}

MoERouting moe_route(const Tensor &x, const Tensor &router_weight, const Tensor *router_bias, const MoEConfig &config)
{
    MoEWeights m;
    m.router_weight = &router_weight;
    m.router_bias = router_bias;
    Checked c = moe_detail::validate(x, m, config, false);
    if (x.device() != Device::CUDA)
        throw std::runtime_error("unsupported device");
    const std::size_t T = c.cfg.num_tokens, E = c.cfg.num_experts, K = c.cfg.top_k;
    MoERouting r;
    r.topk_ids.resize(T * K);
    r.topk_weights.resize(T * K);
    r.counts.resize(E);
    r.offsets.resize(E + 1);
    r.perm.resize(T * K);
    r.inv.resize(T * K);
    if (T == 0)
        return r;
    std::size_t need = 0;
    raise_if(xs_moe_workspace_bytes(&c.cfg, &need));
    Workspace ws(need);
    Tensor ids({(std::int64_t)T, (std::int64_t)K}, DType::Int32, Device::CUDA), tw({(std::int64_t)T, (std::int64_t)K}, DType::Float32, Device::CUDA);
    Tensor counts({(std::int64_t)E}, DType::Int32, Device::CUDA), offsets({(std::int64_t)E + 1}, DType::Int32, Device::CUDA);
    Tensor perm({(std::int64_t)(T * K)}, DType::Int32, Device::CUDA), inv({(std::int64_t)(T * K)}, DType::Int32, Device::CUDA);
    raise_if(xs_moe_route(&c.cfg, x.data(), c.w.router_w_dev, c.w.router_bias_dev, nullptr, ids.data<int32_t>(), tw.data<float>(),
                          ws.data(), ws.bytes(), nullptr));
    raise_if(xs_moe_permute(&c.cfg, ids.data<int32_t>(), counts.data<int32_t>(), offsets.data<int32_t>(), perm.data<int32_t>(),
                            inv.data<int32_t>(), ws.data(), ws.bytes(), nullptr));
    raise_if(xs_moe_check_flags(ws.data(), nullptr));
    cuda_memcpy_d2h(r.topk_ids.data(), ids.data(), ids.nbytes());
    cuda_memcpy_d2h(r.topk_weights.data(), tw.data(), tw.nbytes());
    cuda_memcpy_d2h(r.counts.data(), counts.data(), counts.nbytes());
    cuda_memcpy_d2h(r.offsets.data(), offsets.data(), offsets.nbytes());
    cuda_memcpy_d2h(r.perm.data(), perm.data(), perm.nbytes());
    cuda_memcpy_d2h(r.inv.data(), inv.data(), inv.nbytes());
    return r;
}
