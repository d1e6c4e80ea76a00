// Python bindings of the two-level (NVLink domain x rail) bookkeeping kernels, csrc/kernels/hier.cu.
//
// Reference counterparts: the torch-tensor wrappers moe_routing_sort / topk_remap / build_recv_src_meta /
// efa_permute of csrc/kernels/efa_kernels.cu:1591-1751. None of the wrappers here synchronises with the host.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "../kernels/api.h"

namespace py = pybind11;

namespace {

#define DXH_CHECK(cond, msg)                                                                   \
    do {                                                                                       \
        if (!(cond)) throw std::invalid_argument(std::string("deepep_efa_b200.hier: ") + (msg)); \
    } while (0)

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("deepep_efa_b200.hier: ") + what + ": " + cudaGetErrorString(e));
    }
}

cudaStream_t stream_of(const torch::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

// member [T, G*P] bool -> (sorted_ids [T*G] (first prefix[G] entries valid), counts [G], prefix [G+1], pos [T, G])
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> routing_sort(const torch::Tensor& member, int ranks_per_group) {
    DXH_CHECK(member.is_cuda() && member.dim() == 2 && member.is_contiguous() && member.scalar_type() == torch::kBool, "member must be a contiguous CUDA bool matrix");
    DXH_CHECK(ranks_per_group >= 1 && member.size(1) % ranks_per_group == 0, "columns must be a multiple of ranks_per_group");
    c10::cuda::CUDAGuard guard(member.device());
    const int T = (int)member.size(0), G = (int)(member.size(1) / ranks_per_group);
    DXH_CHECK(G <= 64, "at most 64 destination groups");
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(member.device());
    auto sorted = torch::empty({(int64_t)T * G}, i32), counts = torch::empty({G}, i32), prefix = torch::empty({G + 1}, i32);
    auto pos = torch::empty({T, G}, i32);
    dx::RoutingSortArgs a{};
    a.member = member.data_ptr<bool>();
    a.num_tokens = T;
    a.num_groups = G;
    a.ranks_per_group = ranks_per_group;
    a.sorted_ids = sorted.data_ptr<int>();
    a.counts = counts.data_ptr<int>();
    a.prefix = prefix.data_ptr<int>();
    a.pos = pos.data_ptr<int>();
    check(dx::launch_routing_sort(a, stream_of(member)), "routing_sort");
    return {sorted, counts, prefix, pos};
}

// -> packed uint8 [S, K*12]
torch::Tensor topk_remap_pack(const torch::Tensor& topk_idx, c10::optional<torch::Tensor> topk_weights, const torch::Tensor& sorted_ids,
                              const torch::Tensor& prefix, int num_entries, int experts_per_group) {
    DXH_CHECK(topk_idx.is_cuda() && topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == torch::kInt64, "topk_idx must be contiguous int64 [T,K]");
    DXH_CHECK(sorted_ids.scalar_type() == torch::kInt32 && sorted_ids.is_contiguous() && sorted_ids.numel() >= num_entries, "sorted_ids must be int32 with at least num_entries entries");
    DXH_CHECK(prefix.scalar_type() == torch::kInt32 && prefix.is_contiguous() && prefix.numel() >= 2, "prefix must be int32 [G+1]");
    c10::cuda::CUDAGuard guard(topk_idx.device());
    const int K = (int)topk_idx.size(1);
    auto packed = torch::empty({num_entries, (int64_t)K * 12}, torch::TensorOptions().dtype(torch::kUInt8).device(topk_idx.device()));
    dx::TopkRemapArgs a{};
    a.topk_idx = topk_idx.data_ptr<int64_t>();
    if (topk_weights.has_value()) {
        DXH_CHECK(topk_weights->scalar_type() == torch::kFloat32 && topk_weights->is_contiguous() && topk_weights->sizes() == topk_idx.sizes(), "topk_weights must be f32 [T,K]");
        a.topk_weights = topk_weights->data_ptr<float>();
    }
    a.sorted_ids = sorted_ids.data_ptr<int>();
    a.prefix = prefix.data_ptr<int>();
    a.num_entries = num_entries;
    a.num_topk = K;
    a.num_groups = (int)prefix.numel() - 1;
    a.experts_per_group = experts_per_group;
    a.packed = packed.data_ptr<uint8_t>();
    check(dx::launch_topk_remap_pack(a, stream_of(topk_idx)), "topk_remap_pack");
    return packed;
}

// -> int32 [n, 2] = (source group, bitmask of local ranks)
torch::Tensor recv_src_meta(const torch::Tensor& recv_prefix, c10::optional<torch::Tensor> is_row_in_local_rank, int num_rows) {
    DXH_CHECK(recv_prefix.is_cuda() && recv_prefix.scalar_type() == torch::kInt32 && recv_prefix.is_contiguous() && recv_prefix.numel() >= 2, "recv_prefix must be CUDA int32 [G+1]");
    c10::cuda::CUDAGuard guard(recv_prefix.device());
    auto meta = torch::empty({num_rows, 2}, torch::TensorOptions().dtype(torch::kInt32).device(recv_prefix.device()));
    dx::RecvSrcMetaArgs a{};
    a.recv_prefix = recv_prefix.data_ptr<int>();
    a.num_rows = num_rows;
    a.num_groups = (int)recv_prefix.numel() - 1;
    if (is_row_in_local_rank.has_value()) {
        DXH_CHECK(is_row_in_local_rank->scalar_type() == torch::kBool && is_row_in_local_rank->is_contiguous() && is_row_in_local_rank->dim() == 2 &&
                      is_row_in_local_rank->size(0) >= num_rows && is_row_in_local_rank->size(1) <= 31, "is_row_in_local_rank must be bool [n, P<=31]");
        a.is_row_in_local_rank = is_row_in_local_rank->data_ptr<bool>();
        a.num_local_ranks = (int)is_row_in_local_rank->size(1);
    }
    a.meta = meta.data_ptr<int>();
    check(dx::launch_recv_src_meta(a, stream_of(recv_prefix)), "recv_src_meta");
    return meta;
}

// segments int64 [n, 3] on the GPU = (src byte offset, dst byte offset, bytes); the caller guarantees the ranges
void segmented_copy(const torch::Tensor& src, torch::Tensor dst, const torch::Tensor& segments) {
    DXH_CHECK(src.is_cuda() && dst.is_cuda() && segments.is_cuda() && src.is_contiguous() && dst.is_contiguous(), "src, dst and segments must be contiguous CUDA tensors");
    DXH_CHECK(segments.scalar_type() == torch::kInt64 && segments.is_contiguous() && segments.dim() == 2 && segments.size(1) == 3, "segments must be int64 [n,3]");
    c10::cuda::CUDAGuard guard(src.device());
    dx::SegmentedCopyArgs a{};
    a.src = static_cast<const uint8_t*>(src.data_ptr());
    a.dst = static_cast<uint8_t*>(dst.data_ptr());
    a.segments = segments.data_ptr<int64_t>();
    a.num_segments = (int)segments.size(0);
    check(dx::launch_segmented_copy(a, stream_of(src)), "segmented_copy");
}

// Layout for a group of `num_ranks` ranks in NVLink domains of `ranks_per_node`:
// (num_tokens_per_rank [R], num_tokens_per_node [R/P], num_tokens_per_expert [E], is_token_in_rank [T,R])
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor> layout_hier(const torch::Tensor& topk_idx, int num_experts, int num_ranks,
                                                                                  int ranks_per_node) {
    DXH_CHECK(topk_idx.is_cuda() && topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == torch::kInt64, "topk_idx must be contiguous CUDA int64 [T,K]");
    DXH_CHECK(num_ranks >= 1 && num_ranks <= 64 && ranks_per_node >= 1 && num_ranks % ranks_per_node == 0, "1 <= num_ranks <= 64 in whole NVLink domains");
    DXH_CHECK(num_experts > 0 && num_experts % num_ranks == 0, "num_experts must be a positive multiple of the number of ranks");
    c10::cuda::CUDAGuard guard(topk_idx.device());
    const int T = (int)topk_idx.size(0), K = (int)topk_idx.size(1), nodes = num_ranks / ranks_per_node;
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(topk_idx.device());
    auto per_rank = torch::empty({num_ranks}, i32), per_node = torch::empty({nodes}, i32), per_expert = torch::empty({num_experts}, i32);
    auto in_rank = torch::empty({T, num_ranks}, i32.dtype(torch::kBool));
    // the ticket word must be zero at launch; a fresh zeroed scratch per call keeps this function stateless
    auto scratch = torch::zeros({(int64_t)dx::layout_scratch_ints(num_experts, num_ranks, T, nodes)}, i32);
    dx::LayoutArgs a{};
    a.topk_idx = topk_idx.data_ptr<int64_t>();
    a.num_tokens = T;
    a.num_topk = K;
    a.num_experts = num_experts;
    a.num_ranks = num_ranks;
    a.num_tokens_per_rank = per_rank.data_ptr<int>();
    a.num_tokens_per_expert = per_expert.data_ptr<int>();
    a.is_token_in_rank = in_rank.data_ptr<bool>();
    a.scratch = scratch.data_ptr<int>();
    a.ranks_per_node = ranks_per_node;
    a.num_tokens_per_node = per_node.data_ptr<int>();
    check(dx::launch_layout(a, stream_of(topk_idx)), "layout_hier");
    return {per_rank, per_node, per_expert, in_rank};
}

}  // namespace

void bind_hier(py::module_& m) {
    m.def("routing_sort", &routing_sort, py::arg("member"), py::arg("ranks_per_group") = 1);
    m.def("topk_remap_pack", &topk_remap_pack, py::arg("topk_idx"), py::arg("topk_weights"), py::arg("sorted_ids"), py::arg("prefix"),
          py::arg("num_entries"), py::arg("experts_per_group"));
    m.def("recv_src_meta", &recv_src_meta, py::arg("recv_prefix"), py::arg("is_row_in_local_rank"), py::arg("num_rows"));
    m.def("segmented_copy", &segmented_copy);
    m.def("layout_hier", &layout_hier);
}
