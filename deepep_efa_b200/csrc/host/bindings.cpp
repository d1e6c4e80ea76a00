// Python bindings (module `_dx`): the host runtime, the host-only helpers (Config, Arena, layouts) and
// one launch function per kernel. Launch functions take LISTS of per-rank arguments: one entry in a
// real multi-process job, one entry per emulated rank in the single-GPU emulation (one cooperative
// launch for all of them). All launches go to the CURRENT torch CUDA stream of the rank's device; the
// Python layer chooses the stream (communication stream, compute stream for hook mode).
//
// Reference counterpart: the pybind module at csrc/deep_ep.cpp:4310-4479 and the host halves of
// get_dispatch_layout / intranode_dispatch / intranode_combine (csrc/deep_ep.cpp:517-1035).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "../kernels/gemm_api.h"
#include "runtime.hpp"

namespace py = pybind11;
using dxh::RuntimeCore;

namespace {

#define DX_CHECK(cond, msg)                                                        \
    do {                                                                           \
        if (!(cond)) throw std::invalid_argument(std::string("deepep_efa_b200: ") + (msg)); \
    } while (0)

struct Runtime {
    std::shared_ptr<RuntimeCore> core;
    cudaStream_t comm_stream = nullptr;
    torch::Tensor layout_scratch;  // grows on demand

    Runtime(int rank, int num_ranks, int64_t num_nvl_bytes, int64_t num_ll_bytes, int device, double timeout_ms, bool mask_on_timeout)
        : core(std::make_shared<RuntimeCore>(rank, num_ranks, (uint64_t)num_nvl_bytes, (uint64_t)num_ll_bytes, device, timeout_ms,
                                             mask_on_timeout)) {}

    py::bytes ipc_handle() const { return py::bytes(core->ipc_handle()); }
    void open_peers(const std::vector<std::string>& handles) { core->open_peers(handles); }
    void set_comm_stream(int64_t s) { comm_stream = reinterpret_cast<cudaStream_t>(s); }

    torch::Tensor alloc_symmetric(std::vector<int64_t> sizes, torch::ScalarType dtype) {
        int64_t numel = 1;
        for (auto s : sizes) numel *= s;
        const uint64_t bytes = (uint64_t)numel * c10::elementSize(dtype);
        const uint64_t off = core->arena_alloc(bytes);
        void* p = reinterpret_cast<char*>(core->base()) + off;
        auto keep = core;
        cudaStream_t comm = comm_stream;
        const int dev = core->device();
        auto deleter = [keep, off, comm, dev](void*) {
            std::vector<cudaStream_t> streams;
            try {
                streams.push_back(c10::cuda::getCurrentCUDAStream(dev).stream());
            } catch (...) {
            }
            if (comm != nullptr) streams.push_back(comm);
            keep->arena_release(off, streams);
        };
        return torch::from_blob(p, sizes, deleter, torch::TensorOptions().dtype(dtype).device(torch::kCUDA, dev));
    }

    // Offset of a tensor inside the symmetric buffer, or -1 when it lives elsewhere.
    int64_t symmetric_offset(const torch::Tensor& t) const {
        if (!t.is_cuda() || !t.is_contiguous()) return -1;
        uint64_t off = 0;
        if (!core->in_symmetric(t.data_ptr(), (uint64_t)t.numel() * t.element_size(), &off)) return -1;
        return (int64_t)off;
    }

    // Tensor view over a fixed range of the symmetric buffer (low-latency region). Not owned.
    torch::Tensor view(int64_t off, std::vector<int64_t> sizes, torch::ScalarType dtype) {
        int64_t numel = 1;
        for (auto s : sizes) numel *= s;
        DX_CHECK(off >= 0 && (uint64_t)off + (uint64_t)numel * c10::elementSize(dtype) <= core->total_bytes(), "view out of the symmetric buffer");
        auto keep = core;
        return torch::from_blob(reinterpret_cast<char*>(core->base()) + off, sizes, [keep](void*) {},
                                torch::TensorOptions().dtype(dtype).device(torch::kCUDA, core->device()));
    }

    std::pair<int, std::vector<int>> wait_recv_counts(int num_local_experts) {
        std::vector<int> per;
        int n;
        {
            py::gil_scoped_release rel;
            n = core->wait_recv_counts(num_local_experts, &per);
        }
        return {n, per};
    }

    void set_mask(int rank_to_mask, bool mask) {
        DX_CHECK(rank_to_mask >= 0 && rank_to_mask < core->num_ranks(), "rank_to_mask out of range");
        const int v = mask ? 1 : 0;
        DX_CUDA_CHECK(cudaMemcpyAsync(&core->control()->ll_mask[rank_to_mask], &v, sizeof(int), cudaMemcpyHostToDevice,
                                      c10::cuda::getCurrentCUDAStream(core->device()).stream()));
        DX_CUDA_CHECK(cudaStreamSynchronize(c10::cuda::getCurrentCUDAStream(core->device()).stream()));
    }
    void query_mask(torch::Tensor out) {
        DX_CHECK(out.is_cuda() && out.scalar_type() == torch::kInt32 && out.numel() >= core->num_ranks(), "mask_status must be int32 [num_ranks] on the GPU");
        DX_CUDA_CHECK(cudaMemcpyAsync(out.data_ptr(), core->control()->ll_mask, sizeof(int) * core->num_ranks(), cudaMemcpyDeviceToDevice,
                                      c10::cuda::getCurrentCUDAStream(core->device()).stream()));
    }
    void clean_mask() {
        DX_CUDA_CHECK(cudaMemsetAsync(core->control()->ll_mask, 0, sizeof(int) * dx::kMaxRanks,
                                      c10::cuda::getCurrentCUDAStream(core->device()).stream()));
    }
};

}  // namespace

// used by fused_bindings.cpp, which cannot name the module-local Runtime class
dxh::RuntimeCore* dx_core_of(py::handle runtime) { return runtime.cast<Runtime*>()->core.get(); }

namespace {

cudaStream_t cur_stream(const Runtime* rt) { return c10::cuda::getCurrentCUDAStream(rt->core->device()).stream(); }

void set_local_peers(std::vector<Runtime*> rts) {
    std::vector<RuntimeCore*> cores;
    for (auto* r : rts) cores.push_back(r->core.get());
    for (auto* r : rts) r->core->set_local_peers(cores);
}

template <typename T>
T* ptr_or_null(const c10::optional<torch::Tensor>& t) {
    return t.has_value() && t->defined() ? reinterpret_cast<T*>(t->data_ptr()) : nullptr;
}

void check_launch(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string(what) + ": launch failed: " + cudaGetErrorString(e));
    }
}

// ---------------------------------------------------------------------------------------------
// layout
// ---------------------------------------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> get_dispatch_layout(Runtime* rt, const torch::Tensor& topk_idx, int num_experts) {
    DX_CHECK(topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == torch::kInt64, "topk_idx must be contiguous int64 [T,K]");
    const int R = rt->core->num_ranks();
    DX_CHECK(num_experts > 0 && num_experts % R == 0, "num_experts must be a positive multiple of the number of ranks");
    c10::cuda::CUDAGuard guard(rt->core->device());
    const int T = (int)topk_idx.size(0), K = (int)topk_idx.size(1);
    auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(topk_idx.device());
    auto per_rank = torch::empty({R}, i32), per_expert = torch::empty({num_experts}, i32);
    auto in_rank = torch::empty({T, R}, i32.dtype(torch::kBool));
    const int64_t need = (int64_t)dx::layout_scratch_ints(num_experts, R, T);
    if (!rt->layout_scratch.defined() || rt->layout_scratch.numel() < need) rt->layout_scratch = torch::zeros({need}, i32);
    dx::LayoutArgs a{};
    a.topk_idx = topk_idx.data_ptr<int64_t>();
    a.num_tokens = T;
    a.num_topk = K;
    a.num_experts = num_experts;
    a.num_ranks = R;
    a.num_tokens_per_rank = per_rank.data_ptr<int>();
    a.num_tokens_per_expert = per_expert.data_ptr<int>();
    a.is_token_in_rank = in_rank.data_ptr<bool>();
    a.scratch = rt->layout_scratch.data_ptr<int>();
    check_launch(dx::launch_layout(a, cur_stream(rt)), "get_dispatch_layout");
    return {per_rank, per_expert, in_rank};
}

// ---------------------------------------------------------------------------------------------
// notify: per rank (num_tokens_per_rank, num_tokens_per_expert, is_token_in_rank)
// returns per rank (rank_prefix_matrix, channel_prefix_matrix, recv_channel_prefix_matrix, send_head)
// ---------------------------------------------------------------------------------------------
using NotifyOut = std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>;
std::vector<NotifyOut> notify(std::vector<Runtime*> rts, std::vector<torch::Tensor> ntpr, std::vector<torch::Tensor> ntpe,
                              std::vector<torch::Tensor> itir, int num_channels, int expert_alignment) {
    const int V = (int)rts.size();
    DX_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)ntpr.size() == V && (int)ntpe.size() == V && (int)itir.size() == V, "notify: one entry per rank");
    DX_CHECK(num_channels >= 1 && num_channels <= dx::kMaxChannels, "num_channels out of range");
    DX_CHECK(expert_alignment >= 1, "expert_alignment must be >= 1");
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::NotifyArgs> args(V);
    std::vector<NotifyOut> outs;
    for (int v = 0; v < V; ++v) {
        Runtime* rt = rts[v];
        const int R = rt->core->num_ranks();
        DX_CHECK(rt->core->available(), "runtime is not synchronised with its peers");
        DX_CHECK(ntpr[v].scalar_type() == torch::kInt32 && ntpr[v].numel() == R && ntpr[v].is_contiguous(), "num_tokens_per_rank must be int32 [R]");
        DX_CHECK(ntpe[v].scalar_type() == torch::kInt32 && ntpe[v].is_contiguous() && ntpe[v].numel() % R == 0, "num_tokens_per_expert must be int32 [E]");
        DX_CHECK(itir[v].scalar_type() == torch::kBool && itir[v].dim() == 2 && itir[v].size(1) == R && itir[v].is_contiguous(), "is_token_in_rank must be bool [T,R]");
        const int E = (int)ntpe[v].numel(), T = (int)itir[v].size(0);
        DX_CHECK(E / R <= dx::kMaxLocalExperts, "too many local experts");
        auto i32 = torch::TensorOptions().dtype(torch::kInt32).device(itir[v].device());
        auto rpm = torch::empty({R, R}, i32), cpm = torch::empty({R, num_channels}, i32), rcpm = torch::empty({R, num_channels}, i32);
        auto send_head = torch::empty({T, R}, i32);
        rt->core->reset_recv_counters(E / R);
        dx::NotifyArgs& a = args[v];
        a.ctx = rt->core->ctx();
        a.num_tokens_per_rank = ntpr[v].data_ptr<int>();
        a.num_tokens_per_expert = ntpe[v].data_ptr<int>();
        a.is_token_in_rank = itir[v].data_ptr<bool>();
        a.num_tokens = T;
        a.num_experts = E;
        a.num_channels = num_channels;
        a.expert_alignment = expert_alignment;
        a.rank_prefix_matrix = rpm.data_ptr<int>();
        a.channel_prefix_matrix = cpm.data_ptr<int>();
        a.recv_channel_prefix_matrix = rcpm.data_ptr<int>();
        a.send_head = send_head.data_ptr<int>();
        dxh::HostWords* hw = reinterpret_cast<dxh::HostWords*>(a.ctx.status);  // status is the first member
        a.host_recv_counter = &hw->recv_counter;
        a.host_expert_counter = hw->expert_counter;
        outs.emplace_back(rpm, cpm, rcpm, send_head);
    }
    check_launch(dx::launch_notify(args.data(), V, cur_stream(rts[0])), "notify");
    return outs;
}

// ---------------------------------------------------------------------------------------------
// dispatch. Per rank tuple:
//  (x, x_scales|None, topk_idx|None, topk_weights|None, send_head, rank_prefix_matrix,
//   recv_x, recv_scales|None, recv_topk_idx|None, recv_topk_weights|None, recv_src_idx)
// ---------------------------------------------------------------------------------------------
c10::optional<torch::Tensor> opt_tensor(const py::handle& h) {
    if (h.is_none()) return c10::nullopt;
    return h.cast<torch::Tensor>();
}

void dispatch(std::vector<Runtime*> rts, std::vector<py::tuple> per_rank, int num_experts, bool quantize, bool round_scale,
              int num_worst_tokens, int num_sms) {
    const int V = (int)rts.size();
    DX_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "dispatch: one entry per rank");
    DX_CHECK(num_sms >= 1, "num_sms must be >= 1");
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::DispatchArgs> args(V);
    for (int v = 0; v < V; ++v) {
        Runtime* rt = rts[v];
        const py::tuple& t = per_rank[v];
        DX_CHECK(t.size() == 11, "dispatch: per-rank tuple must have 11 entries");
        const int R = rt->core->num_ranks();
        auto x = t[0].cast<torch::Tensor>();
        auto x_scales = opt_tensor(t[1]);
        auto topk_idx = opt_tensor(t[2]);
        auto topk_w = opt_tensor(t[3]);
        auto send_head = t[4].cast<torch::Tensor>();
        auto rpm = t[5].cast<torch::Tensor>();
        auto recv_x = t[6].cast<torch::Tensor>();
        auto recv_scales = opt_tensor(t[7]);
        auto recv_topk_idx = opt_tensor(t[8]);
        auto recv_topk_w = opt_tensor(t[9]);
        auto recv_src_idx = t[10].cast<torch::Tensor>();
        DX_CHECK(x.dim() == 2 && x.is_contiguous(), "x must be contiguous [T,hidden]");
        const int T = (int)x.size(0), H = (int)x.size(1);
        DX_CHECK((H * x.element_size()) % 16 == 0, "hidden bytes must be a multiple of 16");
        DX_CHECK(send_head.scalar_type() == torch::kInt32 && send_head.is_contiguous() && send_head.size(0) == T && send_head.size(1) == R, "send_head must be int32 [T,R]");
        DX_CHECK(rpm.scalar_type() == torch::kInt32 && rpm.is_contiguous() && rpm.numel() == R * R, "rank_prefix_matrix must be int32 [R,R]");
        dx::DispatchArgs& a = args[v];
        a.ctx = rt->core->ctx();
        a.x = x.data_ptr();
        a.x_elem_bytes = (int)x.element_size();
        a.x_scales = nullptr;
        a.quantize = quantize ? 1 : 0;
        a.round_scale = round_scale ? 1 : 0;
        if (quantize) {
            DX_CHECK(x.scalar_type() == torch::kBFloat16 && H % 128 == 0 && H <= 8192, "fused FP8 dispatch needs bf16 x with hidden % 128 == 0 and hidden <= 8192");
            DX_CHECK(recv_scales.has_value(), "fused FP8 dispatch needs a recv_scales output");
        } else if (x_scales.has_value()) {
            DX_CHECK(x.element_size() == 1 && x_scales->scalar_type() == torch::kFloat32 && x_scales->is_contiguous() && x_scales->size(0) == T, "x_scales must be f32 [T,hidden/128]");
            DX_CHECK(H % 128 == 0 && x_scales->size(1) == H / 128, "x_scales must have hidden/128 columns");
            a.x_scales = x_scales->data_ptr<float>();
        } else {
            DX_CHECK(x.scalar_type() == torch::kBFloat16, "x must be bf16 (or an (e4m3, scales) pair)");
        }
        a.topk_idx = nullptr;
        a.topk_weights = nullptr;
        a.num_topk = 0;
        if (topk_idx.has_value()) {
            DX_CHECK(topk_idx->scalar_type() == torch::kInt64 && topk_idx->is_contiguous() && topk_idx->size(0) == T, "topk_idx must be int64 [T,K]");
            a.num_topk = (int)topk_idx->size(1);
            DX_CHECK(a.num_topk <= dx::kMaxTopk, "num_topk too large");
            a.topk_idx = topk_idx->data_ptr<int64_t>();
            DX_CHECK(recv_topk_idx.has_value(), "recv_topk_idx output missing");
            if (topk_w.has_value()) {
                DX_CHECK(topk_w->scalar_type() == torch::kFloat32 && topk_w->is_contiguous() && topk_w->numel() == topk_idx->numel(), "topk_weights must be f32 [T,K]");
                a.topk_weights = topk_w->data_ptr<float>();
                DX_CHECK(recv_topk_w.has_value(), "recv_topk_weights output missing");
            }
        }
        a.send_head = send_head.data_ptr<int>();
        a.rank_prefix_matrix = rpm.data_ptr<int>();
        a.num_tokens = T;
        a.hidden = H;
        a.num_experts = num_experts;
        a.num_sms = num_sms;
        auto off_of = [&](const torch::Tensor& tt, const char* name) -> uint64_t {
            const int64_t off = rt->symmetric_offset(tt);
            DX_CHECK(off >= 0, std::string(name) + " must live in this rank's symmetric buffer");
            return (uint64_t)off;
        };
        a.recv_x_off = off_of(recv_x, "recv_x");
        a.recv_scales_off = recv_scales.has_value() ? off_of(*recv_scales, "recv_scales") : 0;
        a.recv_topk_idx_off = recv_topk_idx.has_value() ? off_of(*recv_topk_idx, "recv_topk_idx") : 0;
        a.recv_topk_w_off = recv_topk_w.has_value() ? off_of(*recv_topk_w, "recv_topk_weights") : 0;
        a.recv_src_idx_off = off_of(recv_src_idx, "recv_src_idx");
        a.num_worst_tokens = num_worst_tokens;
    }
    check_launch(dx::launch_dispatch(args.data(), V, cur_stream(rts[0])), "dispatch");
}

// ---------------------------------------------------------------------------------------------
// combine. Per rank tuple: (x_sym, topk_weights_sym|None, send_head, rank_prefix_matrix, bias0|None,
//                           bias1|None, out, out_topk_weights|None)
// ---------------------------------------------------------------------------------------------
void combine(std::vector<Runtime*> rts, std::vector<py::tuple> per_rank, int num_sms) {
    const int V = (int)rts.size();
    DX_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "combine: one entry per rank");
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::CombineArgs> args(V);
    for (int v = 0; v < V; ++v) {
        Runtime* rt = rts[v];
        const py::tuple& t = per_rank[v];
        DX_CHECK(t.size() == 8, "combine: per-rank tuple must have 8 entries");
        const int R = rt->core->num_ranks();
        auto x = t[0].cast<torch::Tensor>();
        auto w = opt_tensor(t[1]);
        auto send_head = t[2].cast<torch::Tensor>();
        auto rpm = t[3].cast<torch::Tensor>();
        auto b0 = opt_tensor(t[4]);
        auto b1 = opt_tensor(t[5]);
        auto out = t[6].cast<torch::Tensor>();
        auto out_w = opt_tensor(t[7]);
        DX_CHECK(x.dim() == 2 && x.scalar_type() == torch::kBFloat16, "combine: x must be bf16 [N,hidden]");
        const int H = (int)x.size(1), T = (int)send_head.size(0);
        DX_CHECK(H % 8 == 0, "hidden must be a multiple of 8");
        DX_CHECK(send_head.scalar_type() == torch::kInt32 && send_head.is_contiguous() && send_head.size(1) == R, "send_head must be int32 [T,R]");
        DX_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.size(0) == T && out.size(1) == H, "out must be bf16 [T,hidden]");
        dx::CombineArgs& a = args[v];
        a.ctx = rt->core->ctx();
        const int64_t xo = rt->symmetric_offset(x);
        DX_CHECK(xo >= 0, "combine: x must live in the symmetric buffer (stage it first)");
        a.x_off = (uint64_t)xo;
        a.topk_w_off = ~0ull;
        a.num_topk = 0;
        a.out_topk_w = nullptr;
        if (w.has_value()) {
            const int64_t wo = rt->symmetric_offset(*w);
            DX_CHECK(wo >= 0 && w->scalar_type() == torch::kFloat32 && w->dim() == 2, "combine: topk_weights must be f32 [N,K] in the symmetric buffer");
            a.topk_w_off = (uint64_t)wo;
            a.num_topk = (int)w->size(1);
            DX_CHECK(out_w.has_value() && out_w->scalar_type() == torch::kFloat32 && out_w->is_contiguous(), "combine: out_topk_weights must be f32");
            a.out_topk_w = out_w->data_ptr<float>();
        }
        a.send_head = send_head.data_ptr<int>();
        a.rank_prefix_matrix = rpm.data_ptr<int>();
        auto bias_ptr = [&](const c10::optional<torch::Tensor>& b) -> const __nv_bfloat16* {
            if (!b.has_value()) return nullptr;
            DX_CHECK(b->scalar_type() == torch::kBFloat16 && b->is_contiguous() && b->size(0) == T && b->size(1) == H, "bias must be bf16 [T,hidden]");
            return reinterpret_cast<const __nv_bfloat16*>(b->data_ptr());
        };
        a.bias0 = bias_ptr(b0);
        a.bias1 = bias_ptr(b1);
        a.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        a.num_tokens = T;
        a.hidden = H;
        a.num_sms = num_sms;
    }
    check_launch(dx::launch_combine(args.data(), V, cur_stream(rts[0])), "combine");
}

void barrier(std::vector<Runtime*> rts) {
    const int V = (int)rts.size();
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::BarrierArgs> args(V);
    for (int v = 0; v < V; ++v) args[v].ctx = rts[v]->core->ctx();
    check_launch(dx::launch_barrier(args.data(), V, cur_stream(rts[0])), "barrier");
}

void timeout_probe(Runtime* rt) {
    c10::cuda::CUDAGuard guard(rt->core->device());
    check_launch(dx::launch_timeout_probe(rt->core->ctx(), rt->core->never_set_flag(), cur_stream(rt)), "timeout_probe");
}

// ---------------------------------------------------------------------------------------------
// FP8 cast
// ---------------------------------------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor> per_token_cast_to_fp8(const torch::Tensor& x, bool round_scale, bool use_ue8m0,
                                                               c10::optional<torch::Tensor> group_counts, int rows_per_group,
                                                               c10::optional<torch::Tensor> out_q, c10::optional<torch::Tensor> out_s,
                                                               c10::optional<torch::Tensor> num_rows_dev, bool atoms) {
    DX_CHECK(x.is_cuda() && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == torch::kBFloat16, "x must be contiguous bf16 [M,hidden] on the GPU");
    const int M = (int)x.size(0), H = (int)x.size(1);
    DX_CHECK(H % 128 == 0 && (!use_ue8m0 || H % 512 == 0), "hidden must be a multiple of 128 (512 for UE8M0 scales)");
    c10::cuda::CUDAGuard guard(x.device());
    auto out = out_q.has_value() ? *out_q : torch::empty({M, H}, x.options().dtype(torch::kFloat8_e4m3fn));
    // atoms: the scales leave as the UE8M0 scale atoms of the natively block-scaled GEMM, uint8 [ceil(M/128), hidden/128, 512]
    DX_CHECK(!atoms || !use_ue8m0, "atoms and use_ue8m0 are two different scale formats");
    torch::Tensor scales = out_s.has_value() ? *out_s
                           : atoms ? torch::empty({(M + 127) / 128, H / 128, 512}, x.options().dtype(torch::kUInt8))
                           : (use_ue8m0 ? torch::empty({M, H / 512}, x.options().dtype(torch::kInt32))
                                        : torch::empty({M, H / 128}, x.options().dtype(torch::kFloat32)));
    DX_CHECK(out.is_cuda() && scales.is_cuda() && out.device() == x.device() && scales.device() == x.device(), "outputs must live on x's GPU");
    DX_CHECK(out.is_contiguous() && out.numel() == (int64_t)M * H && out.element_size() == 1, "out_q must be a contiguous 1-byte [M,hidden] tensor");
    if (atoms)
        DX_CHECK(scales.is_contiguous() && scales.element_size() == 1 && scales.numel() >= (int64_t)((M + 127) / 128) * (H / 128) * 512, "out_s must be uint8 [ceil(M/128), hidden/128, 512]");
    else
        DX_CHECK(scales.is_contiguous() && scales.numel() == (int64_t)M * (use_ue8m0 ? H / 512 : H / 128) && scales.element_size() == 4, "out_s has the wrong shape");
    dx::Fp8CastArgs a{};
    a.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
    a.out = reinterpret_cast<uint8_t*>(out.data_ptr());
    a.scales = (use_ue8m0 || atoms) ? nullptr : scales.data_ptr<float>();
    a.scales_ue8m0 = use_ue8m0 ? scales.data_ptr<int32_t>() : nullptr;
    a.sf_atoms = atoms ? scales.data_ptr<uint8_t>() : nullptr;
    if (num_rows_dev.has_value()) {
        DX_CHECK(num_rows_dev->is_cuda() && num_rows_dev->device() == x.device() && num_rows_dev->scalar_type() == torch::kInt32 && num_rows_dev->numel() >= 1,
                 "num_rows_dev must be an int32 tensor on x's GPU");
        a.num_rows_dev = num_rows_dev->data_ptr<int>();
    }
    a.num_rows = M;
    a.hidden = H;
    a.round_scale = round_scale ? 1 : 0;
    a.ue8m0 = use_ue8m0 ? 1 : 0;
    a.group_counts = nullptr;
    a.rows_per_group = 1;
    if (group_counts.has_value()) {
        DX_CHECK(group_counts->is_cuda() && group_counts->scalar_type() == torch::kInt32 && group_counts->is_contiguous() && rows_per_group > 0 &&
                     group_counts->numel() * (int64_t)rows_per_group == M, "group_counts must be int32 [M / rows_per_group]");
        a.group_counts = group_counts->data_ptr<int>();
        a.rows_per_group = rows_per_group;
    }
    check_launch(dx::launch_fp8_cast(a, c10::cuda::getCurrentCUDAStream(x.device().index()).stream()), "per_token_cast_to_fp8");
    return {out, scales};
}

// ---------------------------------------------------------------------------------------------
// low latency
// ---------------------------------------------------------------------------------------------
dx::LLRegion make_region(const dxh::LowLatencyLayout& l) {
    dx::LLRegion r;
    for (int p = 0; p < 2; ++p) {
        r.counts_off[p] = l.counts_off[p];
        r.recv_x_off[p] = l.recv_x_off[p];
        r.recv_scales_off[p] = l.recv_scales_off[p];
        r.recv_src_info_off[p] = l.recv_src_info_off[p];
        r.combine_stage_off[p] = l.combine_stage_off[p];
        r.combine_src_off[p] = l.combine_src_off[p];
    }
    return r;
}

// Per rank tuple: (x, topk_idx, packed_recv_count, layout_range, cumulative_stats|None, wait_stats|None, send_row|None)
void ll_dispatch(std::vector<Runtime*> rts, std::vector<py::tuple> per_rank, int num_max_tokens, int num_experts, bool use_fp8,
                 bool round_scale, bool use_ue8m0, int parity, int phases, int num_sms) {
    const int V = (int)rts.size();
    DX_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "ll_dispatch: one entry per rank");
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::LLDispatchArgs> args(V);
    for (int v = 0; v < V; ++v) {
        Runtime* rt = rts[v];
        const py::tuple& t = per_rank[v];
        DX_CHECK(t.size() == 7, "ll_dispatch: per-rank tuple must have 7 entries");
        auto x = t[0].cast<torch::Tensor>();
        auto topk_idx = t[1].cast<torch::Tensor>();
        auto count = t[2].cast<torch::Tensor>();
        auto range = t[3].cast<torch::Tensor>();
        auto cum = opt_tensor(t[4]);
        auto wait = opt_tensor(t[5]);
        auto slot = opt_tensor(t[6]);
        const int R = rt->core->num_ranks();
        // x may also sit in pinned host memory: the token CTAs then read their rows over PCIe themselves (each row is read
        // exactly once), which is the host-to-device transfer without a copy in front of the kernel
        const bool x_on_gpu = x.is_cuda() && x.device().index() == rt->core->device();
        const bool x_pinned = x.device().is_cpu() && x.is_pinned();
        DX_CHECK((x_on_gpu || x_pinned) && x.dim() == 2 && x.is_contiguous() && x.scalar_type() == torch::kBFloat16,
                 "x must be contiguous bf16 [T,hidden] on this rank's GPU or in pinned host memory");
        DX_CHECK(topk_idx.is_cuda() && topk_idx.device().index() == rt->core->device() && count.is_cuda() && range.is_cuda(),
                 "low_latency_dispatch: every tensor but x must live on this rank's GPU");
        const int T = (int)x.size(0), H = (int)x.size(1);
        DX_CHECK(T <= num_max_tokens, "more tokens than num_max_dispatch_tokens_per_rank");
        DX_CHECK(num_max_tokens <= 65535, "num_max_dispatch_tokens_per_rank must fit the 16-bit count field of the count exchange");
        DX_CHECK((int64_t)R * num_max_tokens < 65535, "rows per expert (ranks x num_max_dispatch_tokens_per_rank) must fit the 16-bit row field of send_row");
        DX_CHECK(H % 128 == 0 && (!use_ue8m0 || H % 512 == 0), "hidden must be a multiple of 128 (512 with UE8M0)");
        DX_CHECK(topk_idx.scalar_type() == torch::kInt64 && topk_idx.is_contiguous() && topk_idx.dim() == 2 && topk_idx.size(0) == T, "topk_idx must be int64 [T,K]");
        DX_CHECK(topk_idx.size(1) <= dx::kMaxTopk, "num_topk too large");
        DX_CHECK(num_experts % R == 0 && count.numel() == num_experts / R && range.numel() == (int64_t)(num_experts / R) * R, "bad output shapes");
        dxh::LowLatencyLayout lay(rt->core->ll_base(), num_max_tokens, H, R, num_experts);
        DX_CHECK(lay.total_bytes <= rt->core->ll_bytes(), "low-latency region too small: create the Buffer with num_rdma_bytes >= get_low_latency_rdma_size_hint(...)");
        dx::LLDispatchArgs& a = args[v];
        a.ctx = rt->core->ctx();
        a.parity = parity;
        a.region = make_region(lay);
        a.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
        a.topk_idx = topk_idx.data_ptr<int64_t>();
        a.num_tokens = T;
        a.hidden = H;
        a.num_topk = (int)topk_idx.size(1);
        a.num_experts = num_experts;
        a.num_max_tokens = num_max_tokens;
        a.use_fp8 = use_fp8;
        a.round_scale = round_scale;
        a.use_ue8m0 = use_ue8m0;
        a.phases = phases;
        a.packed_recv_count = count.data_ptr<int>();
        a.layout_range = range.data_ptr<int64_t>();
        a.cumulative_stats = ptr_or_null<int>(cum);
        a.wait_cost_stats = ptr_or_null<int64_t>(wait);
        if (slot.has_value())
            DX_CHECK(slot->is_cuda() && slot->scalar_type() == torch::kInt32 && slot->is_contiguous() && slot->numel() >= (int64_t)T * topk_idx.size(1), "send_row must be int32 [T,K] on the GPU");
        a.send_row = ptr_or_null<int>(slot);
        a.num_sms = num_sms;
    }
    check_launch(dx::launch_ll_dispatch(args.data(), V, cur_stream(rts[0])), "low_latency_dispatch");
}

// Per rank tuple: (x, topk_idx, topk_weights, src_info, layout_range, out, wait_stats|None, send_row|None)
// pull: x of every rank lives in its symmetric buffer and send_row comes from the dispatch of the same handle; the home
// ranks read the rows in place. close_barrier: readers report back before the kernel ends (x is not the zero-copy buffer).
void ll_combine(std::vector<Runtime*> rts, std::vector<py::tuple> per_rank, int num_max_tokens, int num_experts, int parity, int phases,
                int num_sms, bool pull, bool close_barrier) {
    const int V = (int)rts.size();
    DX_CHECK(V >= 1 && V <= dx::kMaxVirtualRanks && (int)per_rank.size() == V, "ll_combine: one entry per rank");
    c10::cuda::CUDAGuard guard(rts[0]->core->device());
    std::vector<dx::LLCombineArgs> args(V);
    for (int v = 0; v < V; ++v) {
        Runtime* rt = rts[v];
        const py::tuple& t = per_rank[v];
        DX_CHECK(t.size() == 8, "ll_combine: per-rank tuple must have 8 entries");
        auto x = t[0].cast<torch::Tensor>();
        auto send_row = opt_tensor(t[7]);
        auto topk_idx = t[1].cast<torch::Tensor>();
        auto topk_w = t[2].cast<torch::Tensor>();
        auto src_info = t[3].cast<torch::Tensor>();
        auto range = t[4].cast<torch::Tensor>();
        auto out = t[5].cast<torch::Tensor>();
        auto wait = opt_tensor(t[6]);
        const int R = rt->core->num_ranks();
        const int L = num_experts / R;
        DX_CHECK(x.is_cuda() && x.dim() == 3 && x.is_contiguous() && x.scalar_type() == torch::kBFloat16 && x.size(0) == L && x.size(1) == (int64_t)R * num_max_tokens, "x must be contiguous bf16 [L, R*max_tokens, hidden] on the GPU");
        DX_CHECK(x.device().index() == rt->core->device() && topk_idx.is_cuda() && topk_w.is_cuda() && src_info.is_cuda() && range.is_cuda() &&
                     topk_idx.device() == x.device() && topk_w.device() == x.device(), "low_latency_combine: inputs must live on this rank's GPU");
        // the result may go to device memory or straight to pinned (page-locked, device-mapped) host memory
        DX_CHECK((out.is_cuda() && out.device() == x.device()) || (out.device().is_cpu() && out.is_pinned()), "out must be on this rank's GPU or in pinned host memory");
        const int H = (int)x.size(2);
        DX_CHECK(topk_idx.scalar_type() == torch::kInt64 && topk_idx.is_contiguous() && topk_idx.dim() == 2, "topk_idx must be int64 [T,K]");
        const int T = (int)topk_idx.size(0);
        DX_CHECK(T <= num_max_tokens && topk_idx.size(1) <= dx::kMaxTopk, "too many tokens or top-k entries");
        DX_CHECK(topk_w.scalar_type() == torch::kFloat32 && topk_w.is_contiguous() && topk_w.numel() == topk_idx.numel(), "topk_weights must be f32 [T,K]");
        DX_CHECK(src_info.scalar_type() == torch::kInt32 && src_info.is_contiguous() && src_info.numel() == (int64_t)L * R * num_max_tokens, "src_info must be int32 [L,N]");
        DX_CHECK(range.scalar_type() == torch::kInt64 && range.is_contiguous() && range.numel() == (int64_t)L * R, "layout_range must be int64 [L,R]");
        DX_CHECK(out.scalar_type() == torch::kBFloat16 && out.is_contiguous() && out.size(0) == T && out.size(1) == H, "out must be bf16 [T,hidden]");
        dxh::LowLatencyLayout lay(rt->core->ll_base(), num_max_tokens, H, R, num_experts);
        DX_CHECK(lay.total_bytes <= rt->core->ll_bytes(), "low-latency region too small");
        dx::LLCombineArgs& a = args[v];
        a.ctx = rt->core->ctx();
        a.parity = parity;
        a.region = make_region(lay);
        a.x = reinterpret_cast<const __nv_bfloat16*>(x.data_ptr());
        a.topk_idx = topk_idx.data_ptr<int64_t>();
        a.topk_weights = topk_w.data_ptr<float>();
        a.src_info = src_info.data_ptr<int>();
        a.layout_range = range.data_ptr<int64_t>();
        a.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
        a.wait_cost_stats = ptr_or_null<int64_t>(wait);
        a.num_tokens = T;
        a.hidden = H;
        a.num_topk = (int)topk_idx.size(1);
        a.num_experts = num_experts;
        a.num_max_tokens = num_max_tokens;
        a.phases = phases;
        a.num_sms = num_sms;
        a.pull = pull ? 1 : 0;
        a.close_barrier = (pull && close_barrier) ? 1 : 0;
        a.x_off = 0;
        a.send_row = nullptr;
        if (pull) {
            const int64_t xo = rt->symmetric_offset(x);
            DX_CHECK(xo >= 0 && xo % 16 == 0, "pull combine: x must live in this rank's symmetric buffer");
            DX_CHECK(send_row.has_value() && send_row->is_cuda() && send_row->scalar_type() == torch::kInt32 && send_row->is_contiguous() &&
                         send_row->numel() >= (int64_t)T * topk_idx.size(1), "pull combine: send_row must be int32 [T,K] on the GPU");
            a.x_off = (uint64_t)xo;
            a.send_row = send_row->data_ptr<int>();
        }
    }
    check_launch(dx::launch_ll_combine(args.data(), V, cur_stream(rts[0])), "low_latency_combine");
}

// Offsets of the low-latency region for the Python layer (views are created there once and cached).
py::dict ll_layout(Runtime* rt, int num_max_tokens, int hidden, int num_experts) {
    dxh::LowLatencyLayout l(rt->core->ll_base(), num_max_tokens, hidden, rt->core->num_ranks(), num_experts);
    py::dict d;
    auto put = [&](const char* k, const uint64_t* v) { d[k] = py::make_tuple((int64_t)v[0], (int64_t)v[1]); };
    put("counts", l.counts_off);
    put("recv_x", l.recv_x_off);
    put("recv_scales", l.recv_scales_off);
    put("recv_src_info", l.recv_src_info_off);
    put("combine_stage", l.combine_stage_off);
    put("combine_src", l.combine_src_off);
    d["total_bytes"] = (int64_t)l.total_bytes;
    d["available_bytes"] = (int64_t)rt->core->ll_bytes();
    return d;
}

}  // namespace

void bind_gemm(py::module_& m);  // gemm_bindings.cpp
void bind_hier(py::module_& m);  // hier_bindings.cpp
void bind_fused(py::module_& m); // fused_bindings.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "deepep_efa_b200 native runtime (sm_100a)";

    py::class_<dxh::Config>(m, "Config")
        .def(py::init<int, int, int, int, int>(), py::arg("num_sms") = 32, py::arg("num_max_nvl_chunked_send_tokens") = 6,
             py::arg("num_max_nvl_chunked_recv_tokens") = 256, py::arg("num_max_rdma_chunked_send_tokens") = 6,
             py::arg("num_max_rdma_chunked_recv_tokens") = 256)
        .def_readwrite("num_sms", &dxh::Config::num_sms)
        .def_readonly("num_max_nvl_chunked_send_tokens", &dxh::Config::num_max_nvl_chunked_send_tokens)
        .def_readonly("num_max_nvl_chunked_recv_tokens", &dxh::Config::num_max_nvl_chunked_recv_tokens)
        .def_readonly("num_max_rdma_chunked_send_tokens", &dxh::Config::num_max_rdma_chunked_send_tokens)
        .def_readonly("num_max_rdma_chunked_recv_tokens", &dxh::Config::num_max_rdma_chunked_recv_tokens)
        .def("get_nvl_buffer_size_hint", &dxh::Config::get_nvl_buffer_size_hint, py::arg("hidden_bytes"), py::arg("num_ranks"),
             py::arg("max_tokens_per_rank") = dxh::kDefaultHintTokens)
        .def("get_rdma_buffer_size_hint", &dxh::Config::get_rdma_buffer_size_hint, py::arg("hidden_bytes"), py::arg("num_ranks"));
    m.def("get_low_latency_rdma_size_hint", &dxh::get_low_latency_rdma_size_hint, py::arg("num_max_dispatch_tokens_per_rank"),
          py::arg("hidden"), py::arg("num_ranks"), py::arg("num_experts"));
    m.attr("CONTROL_BYTES") = (int64_t)dxh::kControlBytes;
    py::class_<dxh::LowLatencyLayout>(m, "LowLatencyLayout")
        .def(py::init<uint64_t, int, int, int, int>(), py::arg("base"), py::arg("num_max_dispatch_tokens_per_rank"), py::arg("hidden"),
             py::arg("num_ranks"), py::arg("num_experts"))
        .def_readonly("total_bytes", &dxh::LowLatencyLayout::total_bytes)
        .def_property_readonly("counts_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.counts_off[0], l.counts_off[1]); })
        .def_property_readonly("recv_x_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.recv_x_off[0], l.recv_x_off[1]); })
        .def_property_readonly("recv_scales_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.recv_scales_off[0], l.recv_scales_off[1]); })
        .def_property_readonly("recv_src_info_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.recv_src_info_off[0], l.recv_src_info_off[1]); })
        .def_property_readonly("combine_stage_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.combine_stage_off[0], l.combine_stage_off[1]); })
        .def_property_readonly("combine_src_off", [](const dxh::LowLatencyLayout& l) { return std::make_pair(l.combine_src_off[0], l.combine_src_off[1]); });

    py::class_<dxh::Arena>(m, "Arena")
        .def(py::init<uint64_t, uint64_t, uint64_t>(), py::arg("base"), py::arg("size"), py::arg("align") = 1024)
        .def("alloc", &dxh::Arena::alloc)
        .def("free", &dxh::Arena::free)
        .def("owns", &dxh::Arena::owns)
        .def_property_readonly("capacity", &dxh::Arena::capacity)
        .def_property_readonly("in_use", &dxh::Arena::in_use)
        .def_property_readonly("high_water", &dxh::Arena::high_water)
        .def_property_readonly("num_free_blocks", &dxh::Arena::num_free_blocks)
        .def_property_readonly("largest_free", &dxh::Arena::largest_free);

    m.def("status_name", [](int code) { return std::string(dxh::status_name(code)); });

    py::class_<Runtime>(m, "Runtime")
        .def(py::init<int, int, int64_t, int64_t, int, double, bool>(), py::arg("rank"), py::arg("num_ranks"), py::arg("num_nvl_bytes"),
             py::arg("num_ll_bytes"), py::arg("device"), py::arg("timeout_ms") = 10000.0, py::arg("mask_on_timeout") = false)
        .def("ipc_handle", &Runtime::ipc_handle)
        .def("open_peers", &Runtime::open_peers)
        .def("set_comm_stream", &Runtime::set_comm_stream)
        .def("alloc_symmetric", &Runtime::alloc_symmetric)
        .def("symmetric_offset", &Runtime::symmetric_offset)
        .def("view", &Runtime::view)
        .def("wait_recv_counts", &Runtime::wait_recv_counts)
        .def("set_mask", &Runtime::set_mask)
        .def("query_mask", &Runtime::query_mask)
        .def("clean_mask", &Runtime::clean_mask)
        .def("set_timeout_ms", [](Runtime& r, double ms) { r.core->set_timeout_ms(ms); })
        .def("set_debug_checks", [](Runtime& r, bool on) { r.core->set_debug_checks(on); })
        .def("debug_checks", [](Runtime& r) { return r.core->debug_checks(); })
        .def("set_debug_extent", [](Runtime& r, int64_t bytes) { r.core->set_debug_extent((uint64_t)bytes); })
        .def("timeout_ms", [](Runtime& r) { return r.core->timeout_ms(); })
        .def("status_code", [](Runtime& r) { return r.core->status_code(); })
        .def("status_string", [](Runtime& r) { return r.core->status_string(); })
        .def("clear_status", [](Runtime& r) { r.core->clear_status(); })
        .def("enable_trace", [](Runtime& r, bool on) { r.core->enable_trace(on); })
        .def("read_trace", [](Runtime& r) { return r.core->read_trace(); })
        .def("reset_control", [](Runtime& r) { r.core->reset_control(); })
        .def("release", [](Runtime& r) { r.core->release(); })
        .def("is_available", [](Runtime& r) { return r.core->available(); })
        .def("rank", [](Runtime& r) { return r.core->rank(); })
        .def("num_ranks", [](Runtime& r) { return r.core->num_ranks(); })
        .def("device", [](Runtime& r) { return r.core->device(); })
        .def("total_bytes", [](Runtime& r) { return (int64_t)r.core->total_bytes(); })
        .def("arena_capacity", [](Runtime& r) { return (int64_t)r.core->arena().capacity(); })
        .def("arena_in_use", [](Runtime& r) { return (int64_t)r.core->arena().in_use(); })
        .def("arena_high_water", [](Runtime& r) { return (int64_t)r.core->arena().high_water(); })
        .def("ll_bytes", [](Runtime& r) { return (int64_t)r.core->ll_bytes(); });

    m.def("set_local_peers", &set_local_peers);
    m.def("get_dispatch_layout", &get_dispatch_layout);
    m.def("notify", &notify);
    m.def("dispatch", &dispatch);
    m.def("combine", &combine);
    m.def("barrier", &barrier);
    m.def("timeout_probe", &timeout_probe);
    m.def("per_token_cast_to_fp8", &per_token_cast_to_fp8, py::arg("x"), py::arg("round_scale") = false, py::arg("use_ue8m0") = false,
          py::arg("group_counts") = py::none(), py::arg("rows_per_group") = 1, py::arg("out_q") = py::none(), py::arg("out_s") = py::none(),
          py::arg("num_rows_dev") = py::none(), py::arg("atoms") = false);
    m.def("ll_dispatch", &ll_dispatch);
    m.def("ll_combine", &ll_combine, py::arg("runtimes"), py::arg("per_rank"), py::arg("num_max_tokens"), py::arg("num_experts"),
          py::arg("parity"), py::arg("phases"), py::arg("num_sms"), py::arg("pull") = false, py::arg("close_barrier") = false);
    m.def("ll_layout", &ll_layout);
    bind_gemm(m);
    bind_hier(m);
    bind_fused(m);
}
