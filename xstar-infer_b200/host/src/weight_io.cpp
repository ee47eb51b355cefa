#include "weight_io.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <stdexcept>

#include "cuda/cuda_allocator.h"

// ---- mapping ---------------------------------------------------------------------------------------------------
MMapFile::MMapFile(const std::string &path)
{
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0)
        throw std::runtime_error("mmap: cannot open " + path + ": " + std::strerror(errno));
    struct stat st {};
    if (::fstat(fd, &st) != 0) {
        const int e = errno;
        ::close(fd);
        throw std::runtime_error("mmap: cannot stat " + path + ": " + std::strerror(e));
    }
    size_ = static_cast<std::size_t>(st.st_size);
    if (size_ > 0) {
        void *p = ::mmap(nullptr, size_, PROT_READ, MAP_SHARED, fd, 0);
        if (p == MAP_FAILED) {
            const int e = errno;
            ::close(fd);
            throw std::runtime_error("mmap: cannot map " + path + ": " + std::strerror(e));
        }
        addr_ = p;
    }
    ::close(fd); // the mapping keeps the file alive
}

MMapFile::~MMapFile()
{
    if (addr_)
        ::munmap(const_cast<void *>(addr_), size_);
}

// ---- header scan -----------------------------------------------------------------------------------------------
namespace {

struct Scanner {
    const char *p;
    const char *end;

    [[noreturn]] void bad(const char *what) const { throw std::runtime_error(std::string("JSON syntax error: ") + what); }
    void ws()
    {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r'))
            p++;
    }
    char peek()
    {
        ws();
        if (p >= end)
            bad("unexpected end of header");
        return *p;
    }
    void expect(char c)
    {
        if (peek() != c)
            bad("unexpected character");
        p++;
    }
    bool accept(char c)
    {
        if (peek() == c) {
            p++;
            return true;
        }
        return false;
    }
    std::string string()
    {
        expect('"');
        const char *b = p;
        while (p < end && *p != '"') {
            const unsigned char c = static_cast<unsigned char>(*p);
            if (c == '\\' || c >= 0x80)
                throw std::runtime_error("backslash or non-ASCII byte in a string");
            p++;
        }
        if (p >= end)
            bad("unterminated string");
        std::string s(b, p);
        p++;
        return s;
    }
    std::uint64_t number()
    {
        ws();
        if (p >= end || *p < '0' || *p > '9')
            bad("expected a non-negative integer");
        std::uint64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            const std::uint64_t d = static_cast<std::uint64_t>(*p - '0');
            if (v > (UINT64_MAX - d) / 10)
                bad("integer overflow");
            v = v * 10 + d;
            p++;
        }
        return v;
    }
    std::vector<std::uint64_t> numbers()
    {
        std::vector<std::uint64_t> out;
        expect('[');
        if (accept(']'))
            return out;
        do
            out.push_back(number());
        while (accept(','));
        expect(']');
        return out;
    }
    // skips one value of any shape: used for "__metadata__" (strings in it may hold anything but a quote)
    void skip_object()
    {
        expect('{');
        int depth = 1;
        bool in_string = false;
        while (p < end && depth > 0) {
            const char c = *p++;
            if (in_string) {
                if (c == '\\' && p < end)
                    p++;
                else if (c == '"')
                    in_string = false;
            } else if (c == '"') {
                in_string = true;
            } else if (c == '{') {
                depth++;
            } else if (c == '}') {
                depth--;
            }
        }
        if (depth != 0)
            bad("unterminated object");
    }
};

DType dtype_of(const std::string &s)
{
    if (s == "F32")
        return DType::Float32;
    if (s == "BF16")
        return DType::BFloat16;
    if (s == "F8_E4M3")
        return DType::Float8E4M3;
    if (s == "U8")
        return DType::UInt8;
    if (s == "I32")
        return DType::Int32;
    throw std::runtime_error("unsupported dtype " + s);
}

} // namespace

std::unordered_map<std::string, TensorMeta> parse_safetensors_header(const MMapFile &file)
{
    if (file.size() < 8)
        throw std::runtime_error("file too small to hold a safetensors header length");
    const unsigned char *base = static_cast<const unsigned char *>(file.addr());
    std::uint64_t header_len = 0;
    for (int i = 7; i >= 0; i--)
        header_len = (header_len << 8) | base[i];
    if (header_len > file.size() - 8)
        throw std::runtime_error("truncated header: the header length exceeds the file");
    const std::size_t data_start = 8 + static_cast<std::size_t>(header_len);
    Scanner sc{reinterpret_cast<const char *>(base + 8), reinterpret_cast<const char *>(base + data_start)};
    std::unordered_map<std::string, TensorMeta> out;
    sc.expect('{');
    if (!sc.accept('}')) {
        do {
            const std::string name = sc.string();
            sc.expect(':');
            if (name == "__metadata__") {
                sc.skip_object();
                continue;
            }
            std::optional<DType> dtype;
            std::optional<std::vector<std::uint64_t>> shape, span;
            sc.expect('{');
            if (!sc.accept('}')) {
                do {
                    const std::string field = sc.string();
                    sc.expect(':');
                    if (field == "dtype")
                        dtype = dtype_of(sc.string());
                    else if (field == "shape")
                        shape = sc.numbers();
                    else if (field == "data_offsets")
                        span = sc.numbers();
                    else
                        sc.bad("unknown field in a tensor descriptor");
                } while (sc.accept(','));
                sc.expect('}');
            }
            if (!dtype || !shape || !span || span->size() != 2)
                throw std::runtime_error("tensor descriptor missing required field (dtype/shape/data_offsets): " + name);
            std::uint64_t numel = 1;
            TensorMeta m;
            for (std::uint64_t d : *shape) {
                if (d != 0 && numel > UINT64_MAX / d)
                    throw std::runtime_error("header inconsistent: shape overflows: " + name);
                numel *= d;
                m.shape.push_back(static_cast<std::int64_t>(d));
            }
            const std::uint64_t begin = (*span)[0], end = (*span)[1];
            if (end < begin || end - begin != numel * dtype_size(*dtype))
                throw std::runtime_error("header inconsistent: data_offsets of " + name + " span " + std::to_string(end - begin) +
                                         " bytes but shape and dtype give " + std::to_string(numel * dtype_size(*dtype)));
            if (end > file.size() - data_start)
                throw std::runtime_error("tensor data out of file bounds: " + name);
            m.offset = data_start + static_cast<std::size_t>(begin);
            m.dtype = *dtype;
            out[name] = std::move(m);
        } while (sc.accept(','));
        sc.expect('}');
    }
    sc.ws();
    if (sc.p != sc.end)
        sc.bad("trailing characters after the header object");
    return out;
}

Tensor make_weight_view(const MMapFile &file, std::size_t offset, std::vector<std::int64_t> shape, DType dtype)
{
    if (offset % dtype_size(dtype) != 0)
        throw std::runtime_error("offset not aligned to dtype size");
    Tensor t(static_cast<const unsigned char *>(file.addr()) + offset, std::move(shape), dtype, Device::CPU);
    if (offset > file.size() || t.nbytes() > file.size() - offset)
        throw std::runtime_error("view exceeds mapping");
    return t;
}

// ---- one MoE layer ---------------------------------------------------------------------------------------------
namespace {

using Meta = std::unordered_map<std::string, TensorMeta>;

const TensorMeta &need(const Meta &meta, const std::string &name)
{
    auto it = meta.find(name);
    if (it == meta.end())
        throw std::runtime_error("missing weight: " + name);
    return it->second;
}

const unsigned char *bytes_of(const MMapFile &f, const TensorMeta &m)
{
    return static_cast<const unsigned char *>(f.addr()) + m.offset;
}

void put(Tensor &dst, std::size_t dst_offset, const void *src, std::size_t n)
{
    unsigned char *d = static_cast<unsigned char *>(dst.data()) + dst_offset;
    if (dst.device() == Device::CUDA)
        cuda_memcpy_h2d(d, src, n);
    else
        std::memcpy(d, src, n);
}

Tensor whole(const MMapFile &f, const TensorMeta &m, DType as, Device device)
{
    Tensor t(m.shape, as, device);
    put(t, 0, bytes_of(f, m), t.nbytes());
    return t;
}

// weight storage kind of the routed experts, from the dtype of the first expert's gate projection
DType expert_kind(DType file_dtype, const std::string &name)
{
    switch (file_dtype) {
    case DType::BFloat16: return DType::BFloat16;
    case DType::Float8E4M3: return DType::Float8E4M3;
    case DType::UInt8: return DType::Float4E2M1x2;
    default: throw std::runtime_error("dtype mismatch: " + name);
    }
}

void check(const TensorMeta &m, DType file_dtype, std::int64_t rows, std::int64_t cols, const std::string &name)
{
    if (m.dtype != file_dtype)
        throw std::runtime_error("dtype mismatch: " + name);
    if (m.shape.size() != 2 || m.shape[0] != rows || m.shape[1] != cols)
        throw std::runtime_error("shape mismatch: " + name);
}

} // namespace

MoeLayerWeights load_moe_layer(const MMapFile &file, const Meta &meta, const std::string &prefix, std::int64_t num_experts,
                               std::int64_t first_expert, std::int64_t expert_count, Device device)
{
    if (num_experts < 1 || first_expert < 0 || expert_count < 1 || first_expert + expert_count > num_experts)
        throw std::runtime_error("expert count mismatch");
    MoeLayerWeights w;
    w.num_experts = num_experts;
    w.first_expert = first_expert;
    w.expert_count = expert_count;

    const TensorMeta &router = need(meta, prefix + ".gate.weight");
    if (router.dtype != DType::BFloat16)
        throw std::runtime_error("dtype mismatch: " + prefix + ".gate.weight");
    if (router.shape.size() != 2 || router.shape[0] != num_experts)
        throw std::runtime_error("expert count mismatch");
    const std::int64_t H = router.shape[1];
    w.hidden = H;
    w.router_weight = whole(file, router, DType::BFloat16, device);
    if (auto it = meta.find(prefix + ".gate.e_score_correction_bias"); it != meta.end()) {
        if (it->second.dtype != DType::Float32)
            throw std::runtime_error("dtype mismatch: " + it->first);
        if (it->second.shape.size() != 1 || it->second.shape[0] != num_experts)
            throw std::runtime_error("shape mismatch: " + it->first);
        w.router_bias = whole(file, it->second, DType::Float32, device);
    }

    auto ename = [&](std::int64_t e, const char *proj, const char *what) {
        return prefix + ".experts." + std::to_string(e) + "." + proj + "_proj." + what;
    };
    const std::string first_name = ename(first_expert, "gate", "weight");
    const TensorMeta &g0 = need(meta, first_name);
    const DType file_dtype = g0.dtype;
    const DType kind = expert_kind(file_dtype, first_name);
    const bool fp4 = kind == DType::Float4E2M1x2, fp8 = kind == DType::Float8E4M3;
    if (g0.shape.size() != 2)
        throw std::runtime_error("shape mismatch: " + first_name);
    const std::int64_t I = g0.shape[0];
    const std::int64_t kdiv = fp4 ? 2 : 1; // packed nibbles: the last dimension counts bytes
    if (g0.shape[1] * kdiv != H || I < 1 || I % kdiv != 0)
        throw std::runtime_error("shape mismatch: " + first_name);
    if ((fp8 && (I % 128 != 0 || H % 128 != 0)) || (fp4 && (I % 32 != 0 || H % 32 != 0)))
        throw std::runtime_error("shape mismatch: " + first_name + " (scale blocks do not divide the matrix)");
    w.intermediate = I;

    const std::int64_t n = expert_count;
    w.gate_up_weight = Tensor({n, 2 * I, H / kdiv}, kind, device);
    w.down_weight = Tensor({n, H, I / kdiv}, kind, device);
    const std::size_t wsz = dtype_size(kind); // bytes per stored element (a packed FP4 byte holds two codes)
    const std::size_t gu_half = static_cast<std::size_t>(I) * (H / kdiv) * wsz, dn = static_cast<std::size_t>(H) * (I / kdiv) * wsz;
    // scales: FP8 f32 per 128 x 128 block, FP4 e8m0 per 32 along K
    const char *scale_name = fp8 ? "weight_scale_inv" : "weight_scale";
    const DType scale_file = fp8 ? DType::Float32 : DType::UInt8, scale_kind = fp8 ? DType::Float32 : DType::UE8M0;
    std::int64_t gs_rows = 0, gs_cols = 0, ds_rows = 0, ds_cols = 0;
    if (fp8) {
        gs_rows = I / 128, gs_cols = H / 128, ds_rows = H / 128, ds_cols = I / 128;
        w.gate_up_scale = Tensor({n, 2 * gs_rows, gs_cols}, scale_kind, device);
        w.down_scale = Tensor({n, ds_rows, ds_cols}, scale_kind, device);
    } else if (fp4) {
        gs_rows = I, gs_cols = H / 32, ds_rows = H, ds_cols = I / 32;
        w.gate_up_scale = Tensor({n, 2 * gs_rows, gs_cols}, scale_kind, device);
        w.down_scale = Tensor({n, ds_rows, ds_cols}, scale_kind, device);
    }
    const std::size_t sz = dtype_size(scale_kind);
    for (std::int64_t i = 0; i < n; i++) {
        const std::int64_t e = first_expert + i;
        const std::string ng = ename(e, "gate", "weight"), nu = ename(e, "up", "weight"), nd = ename(e, "down", "weight");
        const TensorMeta &g = need(meta, ng), &u = need(meta, nu), &d = need(meta, nd);
        check(g, file_dtype, I, H / kdiv, ng);
        check(u, file_dtype, I, H / kdiv, nu);
        check(d, file_dtype, H, I / kdiv, nd);
        put(w.gate_up_weight, (2 * i) * gu_half, bytes_of(file, g), gu_half); // rows [gate; up], as the dense model fuses them
        put(w.gate_up_weight, (2 * i + 1) * gu_half, bytes_of(file, u), gu_half);
        put(w.down_weight, i * dn, bytes_of(file, d), dn);
        if (fp8 || fp4) {
            const std::string sg = ename(e, "gate", scale_name), su = ename(e, "up", scale_name), sd = ename(e, "down", scale_name);
            const TensorMeta &mg = need(meta, sg), &mu = need(meta, su), &md = need(meta, sd);
            check(mg, scale_file, gs_rows, gs_cols, sg);
            check(mu, scale_file, gs_rows, gs_cols, su);
            check(md, scale_file, ds_rows, ds_cols, sd);
            const std::size_t gsz = static_cast<std::size_t>(gs_rows) * gs_cols * sz, dsz = static_cast<std::size_t>(ds_rows) * ds_cols * sz;
            put(*w.gate_up_scale, (2 * i) * gsz, bytes_of(file, mg), gsz);
            put(*w.gate_up_scale, (2 * i + 1) * gsz, bytes_of(file, mu), gsz);
            put(*w.down_scale, i * dsz, bytes_of(file, md), dsz);
        }
    }

    // the always-on expert: bf16 next to bf16 experts, FP8 128 x 128 next to FP8 and FP4 experts
    const std::string sp = prefix + ".shared_experts.";
    if (meta.count(sp + "gate_proj.weight")) {
        const TensorMeta &g = need(meta, sp + "gate_proj.weight"), &u = need(meta, sp + "up_proj.weight"), &d = need(meta, sp + "down_proj.weight");
        const DType sk = g.dtype;
        if (sk != DType::BFloat16 && sk != DType::Float8E4M3)
            throw std::runtime_error("dtype mismatch: " + sp + "gate_proj.weight");
        check(g, sk, I, H, sp + "gate_proj.weight");
        check(u, sk, I, H, sp + "up_proj.weight");
        check(d, sk, H, I, sp + "down_proj.weight");
        w.shared_gate_up_weight = Tensor({2 * I, H}, sk, device);
        w.shared_down_weight = Tensor({H, I}, sk, device);
        const std::size_t half = static_cast<std::size_t>(I) * H * dtype_size(sk);
        put(*w.shared_gate_up_weight, 0, bytes_of(file, g), half);
        put(*w.shared_gate_up_weight, half, bytes_of(file, u), half);
        put(*w.shared_down_weight, 0, bytes_of(file, d), half);
        if (sk == DType::Float8E4M3) {
            if (I % 128 != 0 || H % 128 != 0)
                throw std::runtime_error("shape mismatch: " + sp + "gate_proj.weight (scale blocks do not divide the matrix)");
            const TensorMeta &mg = need(meta, sp + "gate_proj.weight_scale_inv"), &mu = need(meta, sp + "up_proj.weight_scale_inv"),
                             &md = need(meta, sp + "down_proj.weight_scale_inv");
            check(mg, DType::Float32, I / 128, H / 128, sp + "gate_proj.weight_scale_inv");
            check(mu, DType::Float32, I / 128, H / 128, sp + "up_proj.weight_scale_inv");
            check(md, DType::Float32, H / 128, I / 128, sp + "down_proj.weight_scale_inv");
            w.shared_gate_up_scale = Tensor({2 * (I / 128), H / 128}, DType::Float32, device);
            w.shared_down_scale = Tensor({H / 128, I / 128}, DType::Float32, device);
            const std::size_t gsz = static_cast<std::size_t>(I / 128) * (H / 128) * 4;
            put(*w.shared_gate_up_scale, 0, bytes_of(file, mg), gsz);
            put(*w.shared_gate_up_scale, gsz, bytes_of(file, mu), gsz);
            put(*w.shared_down_scale, 0, bytes_of(file, md), gsz);
        }
    }
    return w;
}
