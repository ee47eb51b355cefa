// Checkpoint IO for the MoE layer: safetensors files mapped read-only, tensors viewed in place, and the experts of one
// layer stacked into the (E, 2I, H) / (E, H, I) tensors the kernels read -- for all experts or for one rank's slice.
//
// Follows the engine's weight IO (reference xstar_cpp/include/weight_io.h:1-56, xstar_cpp/include/mmap_file.h:1-36): a
// whole-file mapping owned by MMapFile, a header scan that returns name -> {offset from file start, shape, dtype}, views
// built by pointer arithmetic, and gate/up fused at load time the way the dense model does it
// (xstar_cpp/src/qwen2_model.cpp:188-206).  The reference knows two storage kinds, F32 and BF16 (weight_io.cpp:122-127); the
// MoE layer adds F8_E4M3 (e4m3 codes), U8 (packed e2m1 codes and e8m0 scales: tagged by the loader, a file cannot tell them
// apart) and I32.
#pragma once
#include <cstdint>
#include <optional>
#include <string>
#include <unordered_map>
#include <vector>

#include "tensor.h"

// Read-only mapping of a whole file; the mapping outlives the descriptor.  Not copyable, not movable: tensor views point
// into it.
class MMapFile
{
public:
    explicit MMapFile(const std::string &path); // throws std::runtime_error("mmap: ...") when the file cannot be mapped
    ~MMapFile();
    MMapFile(const MMapFile &) = delete;
    MMapFile &operator=(const MMapFile &) = delete;
    const void *addr() const { return addr_; }
    std::size_t size() const { return size_; }

private:
    const void *addr_ = nullptr;
    std::size_t size_ = 0;
};

struct TensorMeta {
    std::size_t offset = 0; // from the start of the FILE (length prefix and header included)
    std::vector<std::int64_t> shape;
    DType dtype = DType::Float32;
};

// Layout: [u64 LE header length][JSON header][tensor data].  The header is a flat object
// {"name": {"dtype": "...", "shape": [...], "data_offsets": [begin, end]}, ...} plus an optional "__metadata__" object,
// which is skipped.  A scanner for exactly that shape, not a JSON parser: strings hold no escapes (a backslash or a
// non-ASCII byte is an error), numbers are non-negative integers.  Errors (std::runtime_error): "file too small",
// "truncated header", "JSON syntax error ...", "backslash or non-ASCII byte in a string", "unsupported dtype X",
// "tensor descriptor missing required field", "header inconsistent: ...", "tensor data out of file bounds".
std::unordered_map<std::string, TensorMeta> parse_safetensors_header(const MMapFile &file);

// Borrowing CPU tensor over the mapped bytes (no copy).  Throws "offset not aligned to dtype size" / "view exceeds mapping".
Tensor make_weight_view(const MMapFile &file, std::size_t offset, std::vector<std::int64_t> shape, DType dtype);

// Names of the tensors of one MoE layer inside a checkpoint, relative to `prefix` (e.g. "model.layers.3.mlp"):
//   <prefix>.gate.weight                              (E, H)  BF16   router
//   <prefix>.gate.e_score_correction_bias             (E)     F32    selection bias, optional
//   <prefix>.experts.<e>.{gate,up,down}_proj.weight   (I, H) (I, H) (H, I): BF16 | F8_E4M3 | U8 (packed e2m1, last dim K/2)
//   <prefix>.experts.<e>.{...}_proj.weight_scale_inv  F32 (rows/128, K/128): FP8 block scales
//   <prefix>.experts.<e>.{...}_proj.weight_scale      U8  (rows, K/32):      e8m0 scales of FP4 experts
//   <prefix>.shared_experts.{gate,up,down}_proj.weight (+ .weight_scale_inv)  the always-on expert, optional
// (the naming of public MoE checkpoints; the reference has no MoE checkpoint to pin it).
struct MoeLayerWeights {
    std::int64_t num_experts = 0, first_expert = 0, expert_count = 0, hidden = 0, intermediate = 0;
    Tensor router_weight;
    std::optional<Tensor> router_bias;
    Tensor gate_up_weight, down_weight; // (count, 2I, H) rows [gate; up], (count, H, I); packed FP4: last dim in bytes
    std::optional<Tensor> gate_up_scale, down_scale;
    std::optional<Tensor> shared_gate_up_weight, shared_down_weight, shared_gate_up_scale, shared_down_scale;
};

// Loads experts [first_expert, first_expert + expert_count) of the layer (an expert-parallel rank's slice; pass 0 and
// num_experts for all of them) and stacks them on `device`: one allocation per stacked tensor, one copy per expert tensor
// straight from the mapping (host to device for Device::CUDA).  Router and always-on expert are loaded whole.
// Errors: "missing weight: <name>", "dtype mismatch: <name>", "shape mismatch: <name>", "expert count mismatch".
MoeLayerWeights load_moe_layer(const MMapFile &file, const std::unordered_map<std::string, TensorMeta> &meta, const std::string &prefix,
                               std::int64_t num_experts, std::int64_t first_expert, std::int64_t expert_count, Device device);
