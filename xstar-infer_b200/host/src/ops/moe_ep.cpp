#include "ops/moe_ep.h"

#include <unistd.h>

#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "cuda/cuda_allocator.h"
#include "ops/moe_checked.h"
#include "xs_moe.h"
#include "xs_moe_comm.h"

using moe_detail::Checked;
using moe_detail::raise_if;

EpUniqueId ep_unique_id()
{
    EpUniqueId id{};
    raise_if(xs_moe_comm_unique_id(id.data()));
    return id;
}

std::int64_t ep_capacity_rows(std::int64_t max_tokens, std::int64_t top_k, int world, double capacity_factor)
{
    if (max_tokens < 0 || top_k < 1 || world < 1 || capacity_factor < 0.0 || !std::isfinite(capacity_factor))
        throw std::runtime_error("bad capacity arguments");
    const std::int64_t worst = static_cast<std::int64_t>(world) * max_tokens * top_k;
    std::int64_t rows = worst;
    if (capacity_factor > 0.0) {
        const double want = std::ceil(capacity_factor * static_cast<double>(max_tokens * top_k));
        rows = want < static_cast<double>(worst) ? static_cast<std::int64_t>(want) : worst;
    }
    rows = (rows + 127) / 128 * 128;
    return rows < 128 ? 128 : rows;
}

namespace {

int format_of_dtype(DType d)
{
    switch (d) {
    case DType::BFloat16: return XS_MOE_BF16;
    case DType::Float8E4M3: return XS_MOE_FP8_BLOCK128;
    case DType::Float4E2M1x2: return XS_MOE_FP4_MX32;
    default: throw std::runtime_error("unsupported dtype");
    }
}

// device memory that frees itself
struct DevBuf {
    void *p = nullptr;
    std::size_t bytes = 0;
    DevBuf() = default;
    explicit DevBuf(std::size_t n) : p(cuda_alloc(n < 256 ? 256 : n)), bytes(n) {}
    ~DevBuf() { cuda_free(p); }
    DevBuf(const DevBuf &) = delete;
    DevBuf &operator=(const DevBuf &) = delete;
    DevBuf(DevBuf &&o) noexcept : p(o.p), bytes(o.bytes) { o.p = nullptr; }
    DevBuf &operator=(DevBuf &&o) noexcept
    {
        if (this != &o) {
            cuda_free(p);
            p = o.p;
            bytes = o.bytes;
            o.p = nullptr;
        }
        return *this;
    }
    template <typename T>
    T *as() const
    {
        return static_cast<T *>(p);
    }
};

// what a rank tells the others about its three exchange buffers
constexpr int kPeerBuffers = 5; // rows, scales, return rows, counts matrix, barrier flags
struct PeerInfo {
    std::int64_t pid;
    std::int32_t device;
    std::int32_t pad;
    std::uint64_t ptr[kPeerBuffers];
    std::uint8_t ipc[kPeerBuffers][XS_MOE_IPC_HANDLE_BYTES];
};

std::uint64_t mix(std::uint64_t h, std::uint64_t v)
{
    h ^= v + 0x9e3779b97f4a7c15ull + (h << 6) + (h >> 2);
    return h;
}

} // namespace

struct EpContext::Impl {
    std::shared_ptr<EpGroup> group;
    int rank = 0, world = 1, device = 0;
    EpShape shape;
    int fmt = XS_MOE_BF16, fmt_shared = XS_MOE_BF16;
    std::int64_t El = 0, capacity = 0, back_rows = 0;
    bool wire_bf16 = false;
    bool fused_return = false; // the down GEMM's epilogue stores the result rows into their source ranks itself
    bool signal = false;       // counts exchange and barriers through peer memory instead of NCCL
    void *comm = nullptr;
    void *side = nullptr, *ev_fork = nullptr, *ev_join = nullptr;
    std::uint64_t steps = 0;
    std::int64_t sh_tokens = 0; // the segment bound the always-on expert's offsets currently hold
    bool abandoned = false;

    // exchange buffers other ranks store into, and every rank's addresses of them as this rank sees them
    DevBuf rows, scales, back, tables, counts_all, flags, epoch;
    std::vector<void *> imported;
    // step scratch
    DevBuf ints, ws_route, ws_grouped, y_grouped, sh_codes, sh_scales, sh_y, ws_shared, topk_w;
    std::size_t ws_route_bytes = 0, ws_grouped_bytes = 0, ws_shared_bytes = 0;
    std::int32_t *ids = nullptr, *counts = nullptr, *offsets = nullptr, *perm = nullptr, *inv = nullptr, *all_counts = nullptr,
                 *dest_base = nullptr, *offsets_local = nullptr, *src_offsets = nullptr, *token = nullptr, *sh_offsets = nullptr;

    XsMoeConfig cfg(std::int64_t T, int format, int first, int count) const
    {
        XsMoeConfig c{};
        c.num_tokens = static_cast<int32_t>(T);
        c.hidden = static_cast<int32_t>(shape.hidden);
        c.num_experts = static_cast<int32_t>(shape.experts);
        c.top_k = static_cast<int32_t>(shape.top_k);
        c.intermediate = static_cast<int32_t>(shape.intermediate);
        c.num_shared = 0;
        c.routed_format = format;
        c.shared_format = format;
        c.local_expert_begin = first;
        c.local_expert_count = count;
        return c;
    }

    void sync_group(std::uint64_t signature)
    {
        if (group)
            group->arrive(rank, signature);
    }

    ~Impl()
    {
        for (void *p : imported)
            xs_moe_ipc_close(p);
        if (comm) {
            if (abandoned || (group && group->broken()))
                xs_moe_comm_abort(comm);
            else
                xs_moe_comm_destroy(comm);
        }
        xs_moe_event_destroy(ev_fork);
        xs_moe_event_destroy(ev_join);
        xs_moe_stream_destroy(side);
    }
};

EpContext::EpContext(std::shared_ptr<EpGroup> group, const EpUniqueId &id, int rank, int world, int device, const EpShape &shape,
                     const EpOptions &options)
    : impl_(new Impl)
{
    Impl &m = *impl_;
    if (world < 1 || world > 32 || rank < 0 || rank >= world)
        throw std::runtime_error("bad rank");
    if (group && group->world() != world)
        throw std::runtime_error("group size mismatch");
    if (shape.max_tokens < 1 || shape.hidden < 1 || shape.experts < 1 || shape.top_k < 1 || shape.top_k > shape.experts || shape.intermediate < 1)
        throw std::runtime_error("shape mismatch");
    if (shape.experts % world != 0)
        throw std::runtime_error("expert count mismatch: experts must divide evenly over ranks");
    m.group = std::move(group);
    m.rank = rank;
    m.world = world;
    m.device = device;
    m.shape = shape;
    m.fmt = format_of_dtype(shape.expert_dtype);
    m.fmt_shared = m.fmt == XS_MOE_FP4_MX32 ? XS_MOE_FP8_BLOCK128 : m.fmt;
    m.El = shape.experts / world;
    m.capacity = ep_capacity_rows(shape.max_tokens, shape.top_k, world, options.capacity_factor);
    m.back_rows = shape.max_tokens * shape.top_k;
    m.wire_bf16 = m.fmt != XS_MOE_BF16;
    if (m.capacity > INT32_MAX || m.back_rows > INT32_MAX)
        throw std::runtime_error("shape mismatch: too many rows for 32-bit row indices");
    cuda_set_device(device);
    raise_if(xs_moe_device_check());

    // every rank must see the same problem before anything collective is started
    std::uint64_t sig = 0x45503031ull;
    for (std::uint64_t v : {static_cast<std::uint64_t>(world), static_cast<std::uint64_t>(shape.max_tokens), static_cast<std::uint64_t>(shape.hidden),
                            static_cast<std::uint64_t>(shape.experts), static_cast<std::uint64_t>(shape.top_k),
                            static_cast<std::uint64_t>(shape.intermediate), static_cast<std::uint64_t>(m.fmt),
                            static_cast<std::uint64_t>(shape.shared), static_cast<std::uint64_t>(m.capacity)})
        sig = mix(sig, v);
    m.sync_group(sig);

    raise_if(xs_moe_comm_create(&m.comm, id.data(), rank, world));
    raise_if(xs_moe_stream_create(&m.side));
    raise_if(xs_moe_event_create(&m.ev_fork));
    raise_if(xs_moe_event_create(&m.ev_join));

    const std::size_t H = shape.hidden, T = shape.max_tokens, K = shape.top_k, E = shape.experts, R = world;
    const std::size_t row_bytes = m.fmt == XS_MOE_BF16 ? H * 2 : H;
    const std::size_t scale_bytes = m.fmt == XS_MOE_BF16 ? 0 : (m.fmt == XS_MOE_FP8_BLOCK128 ? (H / 128) * 4 : H / 32);
    m.rows = DevBuf(m.capacity * row_bytes);
    m.scales = DevBuf(m.capacity * scale_bytes);
    m.back = DevBuf(m.back_rows * H * (m.wire_bf16 ? 2 : 4));
    m.tables = DevBuf(kPeerBuffers * R * sizeof(void *));
    m.counts_all = DevBuf(R * E * 4);
    m.flags = DevBuf(R * 4);
    m.epoch = DevBuf(4);
    raise_if(xs_moe_memset_async(m.counts_all.p, 0, R * E * 4, nullptr));
    raise_if(xs_moe_memset_async(m.flags.p, 0, 256, nullptr));
    raise_if(xs_moe_memset_async(m.epoch.p, 0, 256, nullptr));
    m.topk_w = DevBuf(T * K * 4);

    // small int arrays carved from one allocation (each 256-byte aligned)
    auto up = [](std::size_t n) { return (n * 4 + 255) / 256 * 256; };
    const std::size_t n_ids = up(T * K), n_e = up(E), n_e1 = up(E + 1), n_re = up(R * E), n_el1 = up(m.El + 1);
    m.ints = DevBuf(4 * n_ids + 2 * n_e + n_e1 + n_re + n_el1 + 3 * 256);
    std::uint8_t *b = m.ints.as<std::uint8_t>();
    auto take = [&](std::size_t bytes) {
        std::int32_t *p = reinterpret_cast<std::int32_t *>(b);
        b += bytes;
        return p;
    };
    m.ids = take(n_ids);
    m.perm = take(n_ids);
    m.inv = take(n_ids);
    (void)take(n_ids);
    m.counts = take(n_e);
    m.dest_base = take(n_e);
    m.offsets = take(n_e1);
    m.all_counts = m.counts_all.as<std::int32_t>(); // an allocation of its own: peers store into it
    m.src_offsets = take(n_re);
    m.offsets_local = take(n_el1);
    m.token = take(256);
    m.sh_offsets = take(256);
    raise_if(xs_moe_memset_async(m.ints.p, 0, m.ints.bytes, nullptr));

    const XsMoeConfig c_route = m.cfg(T, m.fmt, 0, static_cast<int>(E));
    raise_if(xs_moe_workspace_bytes(&c_route, &m.ws_route_bytes));
    m.ws_route = DevBuf(m.ws_route_bytes);
    raise_if(xs_moe_workspace_init(m.ws_route.p, m.ws_route_bytes, nullptr));
    const XsMoeConfig c_local = m.cfg(T, m.fmt, static_cast<int>(rank * m.El), static_cast<int>(m.El));
    raise_if(xs_moe_grouped_mlp_workspace_bytes(&c_local, static_cast<int32_t>(m.capacity), &m.ws_grouped_bytes));
    m.ws_grouped = DevBuf(m.ws_grouped_bytes);
    raise_if(xs_moe_workspace_init(m.ws_grouped.p, m.ws_grouped_bytes, nullptr));
    std::int32_t fused = 0;
    raise_if(xs_moe_grouped_mlp_return_supported(&c_local, static_cast<int32_t>(m.capacity), &fused));
    m.fused_return = fused != 0 && m.wire_bf16 && options.fused_return;
    if (!m.fused_return)
        m.y_grouped = DevBuf(static_cast<std::size_t>(m.capacity) * H * 4);
    if (shape.shared) {
        const XsMoeConfig c_sh = m.cfg(T, m.fmt_shared, 0, 1);
        raise_if(xs_moe_grouped_mlp_workspace_bytes(&c_sh, static_cast<int32_t>(T), &m.ws_shared_bytes));
        m.ws_shared = DevBuf(m.ws_shared_bytes);
        raise_if(xs_moe_workspace_init(m.ws_shared.p, m.ws_shared_bytes, nullptr));
        m.sh_y = DevBuf(T * H * 4);
        if (m.fmt_shared == XS_MOE_FP8_BLOCK128) {
            m.sh_codes = DevBuf(T * H);
            m.sh_scales = DevBuf(T * (H / 128) * 4);
        }
    }

    // Addresses of every rank's exchange buffers: raw pointers between ranks of one process (after enabling peer access),
    // IPC mappings between processes.  The records travel through an all-gather on the new communicator.
    PeerInfo mine{};
    mine.pid = static_cast<std::int64_t>(getpid());
    mine.device = device;
    void *bufs[kPeerBuffers] = {m.rows.p, m.scales.p, m.back.p, m.counts_all.p, m.flags.p};
    for (int i = 0; i < kPeerBuffers; i++) {
        mine.ptr[i] = reinterpret_cast<std::uint64_t>(bufs[i]);
        raise_if(xs_moe_ipc_export(bufs[i], mine.ipc[i]));
    }
    DevBuf send(sizeof(PeerInfo)), recv(sizeof(PeerInfo) * R);
    cuda_memcpy_h2d(send.p, &mine, sizeof(mine));
    raise_if(xs_moe_comm_all_gather(m.comm, send.p, recv.p, sizeof(PeerInfo), nullptr));
    raise_if(xs_moe_stream_synchronize(nullptr));
    std::vector<PeerInfo> all(R);
    cuda_memcpy_d2h(all.data(), recv.p, sizeof(PeerInfo) * R);
    std::vector<void *> table(kPeerBuffers * R, nullptr);
    bool distinct_devices = true; // two ranks on one GPU (virtual ranks) must not wait for each other inside kernels
    for (std::size_t a = 0; a < R; a++)
        for (std::size_t b2 = a + 1; b2 < R; b2++)
            if (all[a].pid == all[b2].pid && all[a].device == all[b2].device)
                distinct_devices = false;
    m.signal = options.signal_barriers && distinct_devices;
    for (std::size_t r = 0; r < R; r++)
        for (int i = 0; i < kPeerBuffers; i++) {
            if (static_cast<int>(r) == rank) {
                table[i * R + r] = bufs[i];
            } else if (all[r].pid == mine.pid) {
                raise_if(xs_moe_enable_peer_access(all[r].device));
                table[i * R + r] = reinterpret_cast<void *>(all[r].ptr[i]);
            } else {
                void *p = nullptr;
                raise_if(xs_moe_ipc_import(all[r].ipc[i], &p));
                m.imported.push_back(p);
                table[i * R + r] = p;
            }
        }
    cuda_memcpy_h2d(m.tables.p, table.data(), table.size() * sizeof(void *));
    const std::int32_t sh_off[2] = {0, static_cast<std::int32_t>(T)};
    cuda_memcpy_h2d(m.sh_offsets, sh_off, sizeof(sh_off));
    m.sh_tokens = static_cast<std::int64_t>(T);
    raise_if(xs_moe_stream_synchronize(nullptr));
    // nobody starts a step before every rank has mapped every buffer
    raise_if(xs_moe_comm_barrier(m.comm, m.token, nullptr));
    raise_if(xs_moe_stream_synchronize(nullptr));
}

EpContext::~EpContext() = default;

int EpContext::rank() const
{
    return impl_->rank;
}
int EpContext::world() const
{
    return impl_->world;
}
std::int64_t EpContext::capacity_rows() const
{
    return impl_->capacity;
}
bool EpContext::fused_return() const
{
    return impl_->fused_return;
}
bool EpContext::signal_barriers() const
{
    return impl_->signal;
}

void EpContext::abandon() noexcept
{
    impl_->abandoned = true;
    if (impl_->group)
        impl_->group->leave(impl_->rank);
}

void EpContext::forward_into(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, Tensor &out, void *stream)
{
    Impl &m = *impl_;
    Checked c = moe_detail::validate(x, weights, config, true, m.El);
    if (x.device() != Device::CUDA || out.device() != Device::CUDA)
        throw std::runtime_error("unsupported device");
    if (out.dtype() != DType::BFloat16 || out.numel() != x.numel())
        throw std::runtime_error("shape mismatch");
    const std::int64_t T = c.cfg.num_tokens;
    if (T > m.shape.max_tokens || c.cfg.hidden != m.shape.hidden || c.cfg.num_experts != m.shape.experts || c.cfg.top_k != m.shape.top_k ||
        c.cfg.intermediate != m.shape.intermediate || c.cfg.routed_format != m.fmt || (c.cfg.num_shared != 0) != m.shape.shared)
        throw std::runtime_error("shape mismatch: the call does not fit the context it was made for");
    if (m.shape.shared && c.cfg.shared_format != m.fmt_shared)
        throw std::runtime_error("dtype mismatch");

    // host-side check-in: nothing of the step is enqueued unless every rank is here with the same step number
    m.sync_group(mix(mix(0x53544550ull, m.steps), static_cast<std::uint64_t>(m.fmt)));
    m.steps++;

    const int R = m.world;
    const XsMoeConfig c_route = m.cfg(T, m.fmt, 0, static_cast<int>(m.shape.experts));
    const XsMoeConfig c_local = m.cfg(T, m.fmt, static_cast<int>(m.rank * m.El), static_cast<int>(m.El));
    float *tw = m.topk_w.as<float>();
    void *const *t_rows = m.tables.as<void *>();
    void *const *t_scales = t_rows + R;
    void *const *t_back = t_rows + 2 * R;

    // always-on expert: needs only x, so it runs on the side stream next to routing and both exchanges
    if (m.shape.shared) {
        raise_if(xs_moe_event_record(m.ev_fork, stream));
        raise_if(xs_moe_stream_wait_event(m.side, m.ev_fork));
        XsMoeConfig c_sh = m.cfg(T, m.fmt_shared, 0, 1);
        XsMoeWeights w_sh{};
        w_sh.router_w_dev = c.w.router_w_dev;
        w_sh.gate_up_w_dev = c.w.shared_gate_up_w_dev;
        w_sh.down_w_dev = c.w.shared_down_w_dev;
        w_sh.gate_up_scale_dev = c.w.shared_gate_up_scale_dev;
        w_sh.down_scale_dev = c.w.shared_down_scale_dev;
        const void *sh_rows = x.data();
        const float *sh_row_scales = nullptr;
        if (m.fmt_shared == XS_MOE_FP8_BLOCK128) {
            raise_if(xs_moe_quantize_rows_fp8(x.data(), static_cast<int32_t>(T), c.cfg.hidden, m.sh_codes.p, m.sh_scales.as<float>(), m.side));
            sh_rows = m.sh_codes.p;
            sh_row_scales = m.sh_scales.as<float>();
        }
        if (T != m.sh_tokens) { // segment [0, T) of the one always-on "expert" (a synchronous copy: only when T changes)
            const std::int32_t off[2] = {0, static_cast<std::int32_t>(T)};
            cuda_memcpy_h2d(m.sh_offsets, off, sizeof(off));
            m.sh_tokens = T;
        }
        raise_if(xs_moe_grouped_mlp(&c_sh, &w_sh, sh_rows, sh_row_scales, m.sh_offsets, static_cast<int32_t>(T), m.sh_y.as<float>(),
                                    m.ws_shared.p, m.ws_shared_bytes, m.side));
        raise_if(xs_moe_event_record(m.ev_join, m.side));
    }

    raise_if(xs_moe_route(&c_route, x.data(), c.w.router_w_dev, c.w.router_bias_dev, nullptr, m.ids, tw, m.ws_route.p, m.ws_route_bytes,
                          stream));
    raise_if(xs_moe_permute(&c_route, m.ids, m.counts, m.offsets, m.perm, m.inv, m.ws_route.p, m.ws_route_bytes, stream));
    void *const *t_counts = t_rows + 3 * R;
    void *const *t_flags = t_rows + 4 * R;
    auto barrier = [&]() {
        if (m.signal)
            raise_if(xs_moe_ep_signal(R, m.rank, nullptr, 0, nullptr, t_flags, m.flags.as<std::int32_t>(), m.epoch.as<std::int32_t>(),
                                      m.ws_route.p, stream));
        else
            raise_if(xs_moe_comm_barrier(m.comm, m.token, stream));
    };
    if (m.signal) // every rank's counts into every rank's matrix, and a barrier
        raise_if(xs_moe_ep_signal(R, m.rank, m.counts, c_route.num_experts, t_counts, t_flags, m.flags.as<std::int32_t>(),
                                  m.epoch.as<std::int32_t>(), m.ws_route.p, stream));
    else
        raise_if(xs_moe_comm_all_gather(m.comm, m.counts, m.all_counts, static_cast<std::size_t>(m.shape.experts) * 4, stream));
    raise_if(xs_moe_ep_plan(m.all_counts, R, c_route.num_experts, m.rank, m.dest_base, m.offsets_local, m.src_offsets, stream));
    raise_if(xs_moe_ep_dispatch(&c_route, R, x.data(), m.ids, m.inv, m.offsets, m.dest_base, t_rows, t_scales,
                                static_cast<int32_t>(m.capacity), m.ws_route.p, stream));
    barrier(); // every rank's rows have landed
    XsMoeWeights w_local = c.w;
    if (m.fused_return) {
        // the down GEMM stores each finished tile's rows into their source ranks: the return trip overlaps the math
        raise_if(xs_moe_grouped_mlp_return(&c_local, &w_local, m.rows.p, m.scales.as<float>(), m.offsets_local, static_cast<int32_t>(m.capacity), R,
                                           m.rank, m.all_counts, m.src_offsets, t_back, static_cast<int32_t>(m.back_rows), m.ws_grouped.p,
                                           m.ws_grouped_bytes, stream));
    } else {
        raise_if(xs_moe_grouped_mlp(&c_local, &w_local, m.rows.p, m.fmt == XS_MOE_BF16 ? nullptr : m.scales.as<float>(), m.offsets_local,
                                    static_cast<int32_t>(m.capacity), m.y_grouped.as<float>(), m.ws_grouped.p, m.ws_grouped_bytes, stream));
        raise_if(xs_moe_ep_return(&c_route, R, m.rank, m.y_grouped.as<float>(), m.all_counts, m.offsets_local, m.src_offsets,
                                  static_cast<int32_t>(m.capacity), t_back, static_cast<int32_t>(m.back_rows), m.wire_bf16 ? 1 : 0,
                                  m.ws_route.p, stream));
    }
    barrier(); // every expert output for this rank's tokens has landed
    const float *shared_y = nullptr;
    if (m.shape.shared) {
        raise_if(xs_moe_stream_wait_event(stream, m.ev_join));
        shared_y = m.sh_y.as<float>();
    }
    if (m.wire_bf16)
        raise_if(xs_moe_combine_bf16_rows(&c_route, m.back.p, m.inv, tw, shared_y, out.data(), stream));
    else
        raise_if(xs_moe_combine(&c_route, m.back.as<float>(), m.inv, tw, shared_y, out.data(), stream));
}

void EpContext::check(void *stream)
{
    Impl &m = *impl_;
    raise_if(xs_moe_stream_synchronize(stream));
    std::int32_t code = 0;
    raise_if(xs_moe_comm_async_error(m.comm, &code));
    if (code != 0)
        throw std::runtime_error(std::string(xs_moe_last_error()));
    raise_if(xs_moe_check_flags(m.ws_route.p, stream));
    raise_if(xs_moe_check_flags(m.ws_grouped.p, stream));
    if (m.shape.shared)
        raise_if(xs_moe_check_flags(m.ws_shared.p, stream));
}

Tensor moe(const Tensor &x, const MoEWeights &weights, const MoEConfig &config, EpContext *ep)
{
    if (!ep)
        return moe(x, weights, config);
    Tensor out = Tensor::result(x.shape(), DType::BFloat16);
    ep->forward_into(x, weights, config, out, nullptr);
    ep->check(nullptr);
    return out;
}
