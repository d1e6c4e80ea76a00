// Python bindings of the expert-major dispatch used by the fused MoE layer (csrc/kernels/fused.cu). Launch functions take
// lists of per-rank arguments like the other collectives: one entry in a real job, one per emulated rank on a single GPU.
//
// The reference has no counterpart: its dispatch is rank-major (csrc/deep_ep.cpp:609-876) and its users permute to
// expert-major order themselves.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "runtime.hpp"

namespace py = pybind11;

namespace {

#define DXF_CHECK(cond, msg)                                                                    \
    do {                                                                                        \
        if (!(cond)) throw std::invalid_argument(std::string("deepep_efa_b200.fused: ") + (msg)); \
    } while (0)

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("deepep_efa_b200.fused: ") + what + ": " + cudaGetErrorString(e));
    }
}

bool i32_on(const torch::Tensor& t, const torch::Device& dev, int64_t min_numel) {
    return t.is_cuda() && t.device() == dev && t.scalar_type() == torch::kInt32 && t.is_contiguous() && t.numel() >= min_numel;
}

}  // namespace

// The Runtime class of the module is local to bindings.cpp; that file exports this accessor to its core.
dxh::RuntimeCore* dx_core_of(py::handle runtime);

namespace {

int64_t sym_off(dxh::RuntimeCore* core, const torch::Tensor& t, const char* name) {
    uint64_t off = 0;
    DXF_CHECK(t.is_cuda() && t.is_contiguous() && core->in_symmetric(t.data_ptr(), (uint64_t)t.numel() * t.element_size(), &off),
              std::string(name) + " must live in this rank's symmetric buffer");
    return (int64_t)off;
}

// Per rank tuple: (topk_idx, recv_x, recv_scales, recv_info, stage, my_counts, sel_list, send_base, unit_start, m_offsets, m_ends, peer_bases)
void em_notify(std::vector<py::object> rts, std::vector<py::tuple> per_rank, int num_experts, int unit_rows) {
    const int V = (int)rts.size();
    DXF_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "em_notify: one entry per rank");
    std::vector<dx::EmNotifyArgs> args(V);
    dxh::RuntimeCore* core0 = dx_core_of(rts[0]);
    c10::cuda::CUDAGuard guard(core0->device());
    for (int v = 0; v < V; ++v) {
        dxh::RuntimeCore* core = dx_core_of(rts[v]);
        const py::tuple& t = per_rank[v];
        DXF_CHECK(t.size() == 12, "em_notify: per-rank tuple must have 12 entries");
        auto topk_idx = t[0].cast<torch::Tensor>();
        auto recv_x = t[1].cast<torch::Tensor>();
        auto recv_scales = t[2].cast<torch::Tensor>();
        auto recv_info = t[3].cast<torch::Tensor>();
        auto stage = t[4].cast<torch::Tensor>();
        auto my_counts = t[5].cast<torch::Tensor>();
        auto sel_list = t[6].cast<torch::Tensor>();
        auto send_base = t[7].cast<torch::Tensor>();
        auto unit_start = t[8].cast<torch::Tensor>();
        auto m_offsets = t[9].cast<torch::Tensor>();
        auto m_ends = t[10].cast<torch::Tensor>();
        auto peer_bases = t[11].cast<torch::Tensor>();
        const int R = core->num_ranks();
        DXF_CHECK(core->available(), "runtime is not synchronised with its peers");
        DXF_CHECK(num_experts >= R && num_experts % R == 0 && num_experts <= dx::kMaxFusedExperts && num_experts / R <= dx::kMaxLocalExperts,
                  "num_experts must be a multiple of the number of ranks and at most 2048");
        DXF_CHECK(topk_idx.is_cuda() && topk_idx.device().index() == core->device() && topk_idx.scalar_type() == torch::kInt64 &&
                      topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.size(1) <= dx::kMaxTopk,
                  "topk_idx must be contiguous int64 [T,K] on this rank's GPU");
        const int64_t T = topk_idx.size(0), K = topk_idx.size(1), L = num_experts / R;
        DXF_CHECK(T * K < (1 << 24), "too many selections per rank (T*K must stay below 2^24)");
        const auto dev = topk_idx.device();
        DXF_CHECK(i32_on(my_counts, dev, num_experts) && i32_on(sel_list, dev, (int64_t)num_experts * T) && i32_on(send_base, dev, num_experts) &&
                      i32_on(unit_start, dev, num_experts + 2) && i32_on(m_offsets, dev, L + 1) && i32_on(m_ends, dev, L),
                  "em_notify: plan tensors must be int32 on this rank's GPU with the documented sizes");
        DXF_CHECK(peer_bases.is_cuda() && peer_bases.device() == dev && peer_bases.element_size() == 8 && peer_bases.is_contiguous() && peer_bases.numel() >= 4 * R,
                  "peer_bases must be 64-bit [4, R]");
        dx::EmNotifyArgs& a = args[v];
        a.ctx = core->ctx();
        a.topk_idx = topk_idx.data_ptr<int64_t>();
        a.num_tokens = (int)T;
        a.num_topk = (int)K;
        a.num_experts = num_experts;
        a.unit_rows = unit_rows;
        DXF_CHECK(recv_x.dim() == 2 && recv_x.element_size() == 1 && recv_info.numel() >= recv_x.size(0), "recv_x must be [rows, hidden] e4m3 with one info word per row");
        a.rows_cap = (int)recv_x.size(0);
        a.recv_x_off = (uint64_t)sym_off(core, recv_x, "recv_x");
        a.recv_scales_off = (uint64_t)sym_off(core, recv_scales, "recv_scales");
        a.recv_info_off = (uint64_t)sym_off(core, recv_info, "recv_info");
        a.stage_off = (uint64_t)sym_off(core, stage, "stage");
        a.my_counts = my_counts.data_ptr<int>();
        a.sel_list = sel_list.data_ptr<int>();
        a.send_base = send_base.data_ptr<int>();
        a.unit_start = unit_start.data_ptr<int>();
        a.unit_counter = unit_start.data_ptr<int>() + num_experts + 1;  // the tensor's last int is the hand-out counter
        a.m_offsets = m_offsets.data_ptr<int>();
        a.m_ends = m_ends.data_ptr<int>();
        a.peer_bases = reinterpret_cast<uint64_t*>(peer_bases.data_ptr());
    }
    check(dx::launch_em_notify(args.data(), V, at::cuda::getCurrentCUDAStream(core0->device()).stream()), "em_notify");
}

// Per rank tuple: (x, my_counts, sel_list, send_base, unit_start, peer_bases, dst_row|None, trace|None, x_scales|None)
// x is bf16 (rows are quantised by the kernel) or, with x_scales, e4m3 rows quantised beforehand (copied as they are).
void em_dispatch(std::vector<py::object> rts, std::vector<py::tuple> per_rank, int num_experts, int num_topk, int unit_rows,
                 bool round_scale, bool native_atoms, int num_sms) {
    const int V = (int)rts.size();
    DXF_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "em_dispatch: one entry per rank");
    DXF_CHECK(num_sms >= 1 && unit_rows >= 1, "num_sms and unit_rows must be positive");
    std::vector<dx::EmDispatchArgs> args(V);
    dxh::RuntimeCore* core0 = dx_core_of(rts[0]);
    c10::cuda::CUDAGuard guard(core0->device());
    for (int v = 0; v < V; ++v) {
        dxh::RuntimeCore* core = dx_core_of(rts[v]);
        const py::tuple& t = per_rank[v];
        DXF_CHECK(t.size() == 9, "em_dispatch: per-rank tuple must have 9 entries");
        auto x = t[0].cast<torch::Tensor>();
        auto my_counts = t[1].cast<torch::Tensor>();
        auto sel_list = t[2].cast<torch::Tensor>();
        auto send_base = t[3].cast<torch::Tensor>();
        auto unit_start = t[4].cast<torch::Tensor>();
        auto peer_bases = t[5].cast<torch::Tensor>();
        const bool prequant = !t[8].is_none();
        DXF_CHECK(x.is_cuda() && x.device().index() == core->device() && x.dim() == 2 && x.is_contiguous() && x.size(1) % 128 == 0 &&
                      (prequant ? x.element_size() == 1 : x.scalar_type() == torch::kBFloat16),
                  "x must be contiguous [T, hidden] on this rank's GPU, hidden % 128 == 0: bf16, or e4m3 together with x_scales");
        const int64_t T = x.size(0);
        const auto dev = x.device();
        DXF_CHECK(i32_on(my_counts, dev, num_experts) && i32_on(sel_list, dev, (int64_t)num_experts * T) && i32_on(send_base, dev, num_experts) &&
                      i32_on(unit_start, dev, num_experts + 2), "em_dispatch: plan tensors do not match");
        DXF_CHECK(peer_bases.is_cuda() && peer_bases.device() == dev && peer_bases.element_size() == 8 && peer_bases.numel() >= 4 * core->num_ranks(), "peer_bases must be 64-bit [4, R]");
        dx::EmDispatchArgs& a = args[v];
        a.ctx = core->ctx();
        a.x = x.data_ptr();
        a.x_scales = nullptr;
        if (prequant) {
            auto xs = t[8].cast<torch::Tensor>();
            DXF_CHECK(xs.is_cuda() && xs.device() == dev && xs.scalar_type() == torch::kFloat32 && xs.is_contiguous() && xs.numel() == T * (x.size(1) / 128),
                      "x_scales must be f32 [T, hidden/128] on x's GPU");
            a.x_scales = xs.data_ptr<float>();
        }
        a.num_tokens = (int)T;
        a.hidden = (int)x.size(1);
        a.num_topk = num_topk;
        a.num_experts = num_experts;
        a.unit_rows = unit_rows;
        a.round_scale = round_scale ? 1 : 0;
        a.native_atoms = native_atoms ? 1 : 0;
        a.my_counts = my_counts.data_ptr<int>();
        a.sel_list = sel_list.data_ptr<int>();
        a.send_base = send_base.data_ptr<int>();
        a.unit_start = unit_start.data_ptr<int>();
        a.unit_counter = unit_start.data_ptr<int>() + num_experts + 1;
        a.peer_bases = reinterpret_cast<const uint64_t*>(peer_bases.data_ptr());
        a.dst_row = nullptr;
        if (!t[6].is_none()) {
            auto dr = t[6].cast<torch::Tensor>();
            DXF_CHECK(i32_on(dr, dev, T * num_topk), "dst_row must be int32 [T*K]");
            a.dst_row = dr.data_ptr<int>();
        }
        a.trace = nullptr;
        if (!t[7].is_none()) {
            auto tr = t[7].cast<torch::Tensor>();
            DXF_CHECK(tr.is_cuda() && tr.device() == dev && tr.element_size() == 8 && tr.numel() >= 2, "trace must be 64-bit [2]");
            a.trace = reinterpret_cast<unsigned long long*>(tr.data_ptr());
        }
        a.num_sms = num_sms;
    }
    check(dx::launch_em_dispatch(args.data(), V, at::cuda::getCurrentCUDAStream(core0->device()).stream()), "em_dispatch");
}

// Views of the expert-major control words of this rank: (arrival counters [kMaxLocalExperts] u64 inside the symmetric
// control block, expected totals [kMaxLocalExperts] u64 in rank-local memory), as int64 tensors that the gated GEMM reads.
std::pair<torch::Tensor, torch::Tensor> em_gate_words(py::object rt) {
    dxh::RuntimeCore* core = dx_core_of(rt);
    auto opts = torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA, core->device());
    auto arrived = torch::from_blob(core->control()->em_arrived, {dx::kMaxLocalExperts}, opts);
    auto expected = torch::from_blob(core->local_seq() + dx::kFusedExpectedWord0, {dx::kMaxLocalExperts}, opts);
    return {arrived, expected};
}

void stage_reduce(const torch::Tensor& stage, const torch::Tensor& out, const torch::Tensor& topk_idx, const torch::Tensor& w, int num_experts) {
    DXF_CHECK(stage.is_cuda() && out.is_cuda() && topk_idx.is_cuda() && w.is_cuda() && stage.device() == out.device() &&
                  topk_idx.device() == out.device() && w.device() == out.device(), "stage_reduce: all tensors on one GPU");
    DXF_CHECK(topk_idx.scalar_type() == torch::kInt64 && topk_idx.dim() == 2 && topk_idx.is_contiguous(), "topk_idx must be int64 [T,K]");
    const int64_t T = topk_idx.size(0), K = topk_idx.size(1);
    DXF_CHECK(out.scalar_type() == torch::kBFloat16 && out.dim() == 2 && out.is_contiguous() && out.size(0) == T, "out must be bf16 [T, hidden]");
    const int64_t H = out.size(1);
    DXF_CHECK(stage.scalar_type() == torch::kBFloat16 && stage.is_contiguous() && stage.numel() >= T * K * H, "stage must be bf16 [T*K, hidden]");
    DXF_CHECK(w.scalar_type() == torch::kFloat32 && w.is_contiguous() && w.numel() == T * K, "weights must be f32 [T,K]");
    c10::cuda::CUDAGuard guard(out.device());
    check(dx::launch_stage_reduce(stage.data_ptr(), out.data_ptr(), topk_idx.data_ptr<int64_t>(), w.data_ptr<float>(), (int)T, (int)K, num_experts,
                                  (int)H, at::cuda::getCurrentCUDAStream(out.device().index()).stream()), "stage_reduce");
}

}  // namespace

void bind_fused(py::module_& m) {
    m.def("em_notify", &em_notify);
    m.def("em_dispatch", &em_dispatch);
    m.def("em_gate_words", &em_gate_words);
    m.def("stage_reduce", &stage_reduce);
}
