// Python bindings of the grouped expert GEMM (kept in its own translation unit so that kernel-side
// changes do not rebuild the runtime bindings).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

#include "../kernels/gemm_api.h"

namespace py = pybind11;

namespace {

#define DXG_CHECK(cond, msg)                                                                  \
    do {                                                                                      \
        if (!(cond)) throw std::invalid_argument(std::string("deepep_efa_b200.grouped_gemm: ") + (msg)); \
    } while (0)

// One error word per device: set by a kernel whose bounded pipeline wait ran out.
torch::Tensor error_flag(int device) {
    static std::mutex mu;
    static std::map<int, torch::Tensor> flags;
    std::lock_guard<std::mutex> g(mu);
    auto it = flags.find(device);
    if (it == flags.end()) {
        auto t = torch::zeros({1}, torch::TensorOptions().dtype(torch::kInt32).device(torch::kCUDA, device));
        it = flags.emplace(device, t).first;
    }
    return it->second;
}

int sm_count(int device) {
    static std::map<int, int> cache;
    auto it = cache.find(device);
    if (it != cache.end()) return it->second;
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device);
    cache[device] = n;
    return n;
}

// SM clock in kHz, cached: this attribute query goes to the driver and costs about a millisecond per call.
int clock_khz(int device) {
    static std::mutex mu;
    static std::map<int, int> cache;
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(device);
    if (it != cache.end()) return it->second;
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
    if (khz <= 0) khz = 1965000;
    cache[device] = khz;
    return khz;
}

// mode 0: a [M,K], b [G,N,K] (or [G*N,K]), m_offsets [G+1] -> c [M, N] (or [M, N/2] with swiglu)
// mode 1: a [N_out, M], b [K_out, M], m_offsets [G+1] -> c [G, N_out, K_out]
torch::Tensor grouped_gemm(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& m_offsets, int mode, bool swiglu,
                           c10::optional<torch::Tensor> a_scales, c10::optional<torch::Tensor> b_scales,
                           c10::optional<torch::Tensor> out, int num_sms, double timeout_ms, c10::optional<torch::Tensor> m_ends,
                           c10::optional<torch::Tensor> sfa_atoms, c10::optional<torch::Tensor> sfb_atoms,
                           c10::optional<torch::Tensor> ready, c10::optional<torch::Tensor> expected,
                           c10::optional<torch::Tensor> row_info, c10::optional<torch::Tensor> scatter_bases,
                           c10::optional<torch::Tensor> trace, bool mn_major, c10::optional<torch::Tensor> out_fp8,
                           c10::optional<torch::Tensor> out_atoms) {
    DXG_CHECK(a.is_cuda() && b.is_cuda() && m_offsets.is_cuda(), "operands must be CUDA tensors");
    DXG_CHECK(a.is_contiguous() && b.is_contiguous() && m_offsets.is_contiguous(), "operands must be contiguous");
    DXG_CHECK(m_offsets.scalar_type() == torch::kInt32 && m_offsets.dim() == 1 && m_offsets.numel() >= 2, "m_offsets must be int32 [G+1]");
    const bool fp8 = a.scalar_type() == torch::kFloat8_e4m3fn;
    DXG_CHECK(fp8 || a.scalar_type() == torch::kBFloat16, "A must be bf16 or float8_e4m3fn");
    DXG_CHECK(b.scalar_type() == a.scalar_type(), "A and B must have the same dtype");
    DXG_CHECK(a.dim() == 2, "A must be 2-D");
    DXG_CHECK((reinterpret_cast<uintptr_t>(a.data_ptr()) & 15) == 0 && (reinterpret_cast<uintptr_t>(b.data_ptr()) & 15) == 0, "operands must be 16-byte aligned");
    const int G = (int)m_offsets.numel() - 1;
    const int device = a.device().index();
    // every operand and output is dereferenced by the kernel on A's device: a host tensor or one from another GPU
    // must be refused here, it would be an illegal address there
    auto same_dev = [&](const c10::optional<torch::Tensor>& t) { return !t.has_value() || (t->is_cuda() && t->device() == a.device()); };
    DXG_CHECK(b.device() == a.device() && m_offsets.device() == a.device(), "A, B and m_offsets must live on the same GPU");
    DXG_CHECK(same_dev(a_scales) && same_dev(b_scales) && same_dev(out) && same_dev(m_ends) && same_dev(sfa_atoms) && same_dev(sfb_atoms) &&
                  same_dev(ready) && same_dev(expected) && same_dev(row_info) && same_dev(scatter_bases) && same_dev(trace),
              "scales, atoms, m_ends, gating / scatter tensors and out must be CUDA tensors on A's device");
    c10::cuda::CUDAGuard guard(device);
    dx::GroupedGemmArgs p{};
    p.num_groups = G;
    p.mode = mode;
    p.fp8 = fp8 ? 1 : 0;
    p.swiglu = swiglu ? 1 : 0;
    torch::Tensor c;
    auto bf16 = a.options().dtype(torch::kBFloat16);
    DXG_CHECK(!mn_major || (!fp8 && !swiglu), "MN-major operands are bf16 only, without swiglu");
    if (mode == 0) {
        const int64_t M = a.size(0), K = a.size(1);
        DXG_CHECK(b.numel() % ((int64_t)G * K) == 0, "B must be [G, N, K]");
        const int64_t N = b.numel() / ((int64_t)G * K);
        // MN-major B is [G, K, N]: the forward weight read as the operand of the input-gradient GEMM
        DXG_CHECK(mn_major ? (b.dim() == 3 && b.size(1) == K && b.size(2) == N) : b.size(-1) == K, "B's reduction dimension must equal K");
        p.b_mn = mn_major ? 1 : 0;
        DXG_CHECK(!swiglu || N % 2 == 0, "swiglu needs an even N (gate and up stacked)");
        const int64_t out_cols = swiglu ? N / 2 : N;
        // with the scatter epilogue nothing is stored to `c`: every row goes to the address its row_info word names
        c = out.has_value() ? *out : torch::empty({(row_info.has_value() || out_fp8.has_value()) ? (int64_t)0 : M, out_cols}, bf16);
        DXG_CHECK(c.scalar_type() == torch::kBFloat16 && c.is_contiguous() && (row_info.has_value() || out_fp8.has_value() || c.numel() == M * out_cols), "out must be contiguous bf16 [M, N]");
        p.m_total = (int)M;
        p.n = (int)N;
        p.k = (int)K;
        if (fp8 && sfa_atoms.has_value()) {
            // native block scaling: pre-built UE8M0 atoms (build_sf_atoms_a / build_sf_atoms_b)
            DXG_CHECK(sfb_atoms.has_value(), "sfa_atoms and sfb_atoms go together");
            DXG_CHECK(K % 128 == 0 && N % 128 == 0, "native block scaling needs K % 128 == 0 and N % 128 == 0");
            DXG_CHECK(!swiglu || (N / 2) % 128 == 0, "native block scaling with swiglu needs N/2 % 128 == 0");
            const int64_t atoms_n = N / 128;  // plain: one atom per 128-row tile; swiglu: two atoms per 256-row tile
            DXG_CHECK(sfa_atoms->is_cuda() && sfa_atoms->scalar_type() == torch::kUInt8 && sfa_atoms->is_contiguous() &&
                          sfa_atoms->numel() >= ((M + 127) / 128) * (K / 128) * 512, "sfa_atoms must be uint8 [ceil(M/128), K/128, 512]");
            DXG_CHECK(sfb_atoms->is_cuda() && sfb_atoms->scalar_type() == torch::kUInt8 && sfb_atoms->is_contiguous() &&
                          sfb_atoms->numel() == (int64_t)G * atoms_n * (K / 128) * 512, "sfb_atoms must be uint8 [G, N/128 atoms, K/128, 512]");
            p.mx_wide = sfb_atoms->size(-1) == 1024 ? 1 : 0;  // the atom layout says which tile width it was built for
            DXG_CHECK(!p.mx_wide || swiglu || N % 256 == 0, "scale atoms built for 256-column tiles need N % 256 == 0");
            p.sfa_atoms = sfa_atoms->data_ptr<uint8_t>();
            p.sfb_atoms = sfb_atoms->data_ptr<uint8_t>();
        } else if (fp8) {
            DXG_CHECK(a_scales.has_value() && b_scales.has_value(), "fp8 operands need a_scales and b_scales");
            DXG_CHECK(a_scales->scalar_type() == torch::kFloat32 && a_scales->is_contiguous() && a_scales->numel() == M * (K / 128), "a_scales must be f32 [M, K/128]");
            DXG_CHECK(b_scales->scalar_type() == torch::kFloat32 && b_scales->is_contiguous() && b_scales->numel() == (int64_t)G * (N / 128) * (K / 128), "b_scales must be f32 [G, N/128, K/128]");
            p.a_scales = a_scales->data_ptr<float>();
            p.b_scales = b_scales->data_ptr<float>();
        }
    } else {
        DXG_CHECK(mode == 1 && !fp8 && !swiglu, "K-grouped mode is bf16 only, without swiglu");
        // ordinary: A [N_out, M], B [K_out, M]; MN-major: A [M, N_out], B [M, K_out] (gradient and activation as they are)
        const int md = mn_major ? 0 : 1;
        DXG_CHECK(b.dim() == 2 && a.size(md) == b.size(md), "mode 1: A and B must share M");
        const int64_t n_out = a.size(1 - md), k_out = b.size(1 - md), M = a.size(md);
        p.a_mn = p.b_mn = mn_major ? 1 : 0;
        c = out.has_value() ? *out : torch::empty({(int64_t)G, n_out, k_out}, bf16);
        DXG_CHECK(c.scalar_type() == torch::kBFloat16 && c.is_contiguous() && c.numel() == (int64_t)G * n_out * k_out, "out must be contiguous bf16 [G, N_out, K_out]");
        p.m_total = (int)M;
        p.n = (int)n_out;
        p.k = (int)k_out;
    }
    p.a = a.data_ptr();
    p.b = b.data_ptr();
    p.c = c.data_ptr();
    p.m_offsets = m_offsets.data_ptr<int>();
    p.m_ends = nullptr;
    if (m_ends.has_value()) {
        DXG_CHECK(mode == 0 && m_ends->is_cuda() && m_ends->scalar_type() == torch::kInt32 && m_ends->is_contiguous() && m_ends->numel() == G, "m_ends must be int32 [G] on the GPU (M-grouped mode only)");
        p.m_ends = m_ends->data_ptr<int>();
    }
    p.num_sms = num_sms > 0 ? num_sms : sm_count(device);
    {
        const char* o = std::getenv("DEEPEP_GEMM_ORDER");
        p.tile_order = (o != nullptr && o[0] == '1') ? 1 : 0;
        // CTA pairs (cta_group::2) pay off for BF16 with about a thousand rows per expert or more (+1-3 % in a power-limited loop); the FP8 path hands a
        // window to the epilogue every K block, and the cross-CTA handshake per block costs more than the halved B traffic saves
        const char* pr = std::getenv("DEEPEP_GEMM_PAIR");
        if (pr != nullptr && (pr[0] == '0' || pr[0] == '1')) p.cta_pairs = pr[0] == '1';
        else p.cta_pairs = (!fp8 && p.m_ends == nullptr && (mode == 1 || (int64_t)p.m_total >= 1024 * (int64_t)G)) ? 1 : 0;
        if (p.num_sms < 2 || mn_major) p.cta_pairs = 0;
        // natively block-scaled e4m3: a pair instantiation exists for the wide SwiGLU tile only
        if (fp8 && !(p.sfa_atoms != nullptr && p.mx_wide == 1)) p.cta_pairs = (pr != nullptr && pr[0] == '1' && p.sfa_atoms == nullptr) ? 1 : 0;
    }
    if (ready.has_value() || expected.has_value()) {
        DXG_CHECK(mode == 0 && ready.has_value() && expected.has_value(), "ready and expected go together (M-grouped mode)");
        DXG_CHECK(ready->element_size() == 8 && expected->element_size() == 8 && ready->is_contiguous() && expected->is_contiguous() &&
                      ready->numel() >= G && expected->numel() >= G, "ready / expected must be 64-bit [G]");
        p.ready = reinterpret_cast<const unsigned long long*>(ready->data_ptr());
        p.expected = reinterpret_cast<const unsigned long long*>(expected->data_ptr());
    }
    if (row_info.has_value() || scatter_bases.has_value()) {
        DXG_CHECK(mode == 0 && !swiglu && row_info.has_value() && scatter_bases.has_value() && m_ends.has_value(),
                  "the scatter epilogue needs row_info, scatter_bases and m_ends (M-grouped mode, no swiglu)");
        DXG_CHECK(row_info->scalar_type() == torch::kInt32 && row_info->is_contiguous() && row_info->numel() >= p.m_total, "row_info must be int32 [M]");
        DXG_CHECK(scatter_bases->element_size() == 8 && scatter_bases->is_contiguous() && scatter_bases->numel() >= 1, "scatter_bases must be 64-bit pointers");
        p.row_info = row_info->data_ptr<int>();
        p.scatter_bases = reinterpret_cast<const unsigned long long*>(scatter_bases->data_ptr());
    }
    if (out_fp8.has_value() || out_atoms.has_value()) {
        DXG_CHECK(out_fp8.has_value() && out_atoms.has_value() && same_dev(out_fp8) && same_dev(out_atoms), "out_fp8 and out_atoms go together, on A's device");
        DXG_CHECK(mode == 0 && swiglu && p.sfa_atoms != nullptr && p.mx_wide == 1, "quantised output needs the natively block-scaled kernel with wide SwiGLU tiles");
        const int64_t inter = p.n / 2;
        DXG_CHECK(out_fp8->element_size() == 1 && out_fp8->is_contiguous() && out_fp8->numel() == (int64_t)p.m_total * inter, "out_fp8 must be e4m3 [M, N/2]");
        DXG_CHECK(out_atoms->element_size() == 1 && out_atoms->is_contiguous() && out_atoms->numel() >= (((int64_t)p.m_total + 127) / 128) * (inter / 128) * 512,
                  "out_atoms must be uint8 [ceil(M/128), N/2/128, 512]");
        p.c_fp8 = reinterpret_cast<uint8_t*>(out_fp8->data_ptr());
        p.c_atoms = reinterpret_cast<uint8_t*>(out_atoms->data_ptr());
    }
    if (trace.has_value()) {
        DXG_CHECK(trace->element_size() == 8 && trace->is_contiguous() && trace->numel() >= 4, "trace must be 64-bit [4]");
        p.trace = reinterpret_cast<unsigned long long*>(trace->data_ptr());
    }
    p.error_flag = error_flag(device).data_ptr<int>();
    p.timeout_cycles = (long long)(timeout_ms * (double)clock_khz(device));
    const cudaError_t e = dx::launch_grouped_gemm(p, at::cuda::getCurrentCUDAStream(device).stream());
    if (e == cudaErrorInvalidValue) {
        cudaGetLastError();
        throw std::invalid_argument(
            "deepep_efa_b200.grouped_gemm: unsupported shape (need K % 64 == 0 for bf16 / % 128 for fp8, N % 128 == 0; the "
            "K-grouped mode needs group boundaries on multiples of 128)");
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        throw std::runtime_error(std::string("deepep_efa_b200.grouped_gemm: launch failed: ") + cudaGetErrorString(e));
    }
    return c;
}

std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> build_plan(const torch::Tensor& topk_idx, const torch::Tensor& m_offsets, int64_t m_pad) {
    DXG_CHECK(topk_idx.is_cuda() && topk_idx.dim() == 2 && topk_idx.is_contiguous() && topk_idx.scalar_type() == torch::kInt64, "topk_idx must be contiguous int64 [N,K] on the GPU");
    DXG_CHECK(m_offsets.is_cuda() && m_offsets.scalar_type() == torch::kInt32 && m_offsets.is_contiguous() && m_offsets.numel() >= 2, "m_offsets must be int32 [L+1] on the GPU");
    const int64_t N = topk_idx.size(0), K = topk_idx.size(1), L = m_offsets.numel() - 1;
    c10::cuda::CUDAGuard guard(topk_idx.device());
    auto i32 = topk_idx.options().dtype(torch::kInt32);
    auto pos = torch::empty({N, K}, i32), src_row = torch::empty({m_pad}, i32), src_k = torch::empty({m_pad}, i32), counters = torch::empty({L}, i32);
    const cudaError_t e = dx::launch_build_plan(topk_idx.data_ptr<int64_t>(), m_offsets.data_ptr<int>(), counters.data_ptr<int>(), pos.data_ptr<int>(),
                                                src_row.data_ptr<int>(), src_k.data_ptr<int>(), (int)N, (int)K, (int)L, (int)m_pad,
                                                at::cuda::getCurrentCUDAStream(topk_idx.device().index()).stream());
    if (e != cudaSuccess) throw std::runtime_error(std::string("build_plan: ") + cudaGetErrorString(e));
    return {pos, src_row, src_k};
}

// dst[m] = scale[m] * src[src_row[m]]; rows of any dtype whose byte size is a multiple of 16
torch::Tensor gather_rows(const torch::Tensor& src, const torch::Tensor& src_row, c10::optional<torch::Tensor> scale,
                          c10::optional<torch::Tensor> out) {
    DXG_CHECK(src.is_cuda() && src.dim() == 2 && src.is_contiguous(), "src must be a contiguous CUDA matrix");
    DXG_CHECK(src_row.scalar_type() == torch::kInt32 && src_row.is_contiguous() && src_row.dim() == 1, "src_row must be int32 [M]");
    const int64_t M = src_row.numel();
    const int64_t row_bytes = src.size(1) * src.element_size();
    DXG_CHECK(row_bytes % 16 == 0, "row size must be a multiple of 16 bytes");
    c10::cuda::CUDAGuard guard(src.device());
    torch::Tensor dst = out.has_value() ? *out : torch::empty({M, src.size(1)}, src.options());
    DXG_CHECK(dst.is_contiguous() && dst.scalar_type() == src.scalar_type() && dst.size(0) == M && dst.size(1) == src.size(1), "out has the wrong shape");
    const float* sc = nullptr;
    if (scale.has_value()) {
        DXG_CHECK(src.scalar_type() == torch::kBFloat16 && scale->scalar_type() == torch::kFloat32 && scale->numel() == M && scale->is_contiguous(), "scale needs bf16 rows and f32 [M]");
        sc = scale->data_ptr<float>();
    }
    const cudaError_t e = dx::launch_gather_rows(src.data_ptr(), dst.data_ptr(), src_row.data_ptr<int>(), sc, (int)M, (int)row_bytes,
                                                 at::cuda::getCurrentCUDAStream(src.device().index()).stream());
    if (e != cudaSuccess) throw std::runtime_error(std::string("gather_rows: ") + cudaGetErrorString(e));
    return dst;
}

// dst[n] = sum_k w[n,k] * src[pos[n,k]]
torch::Tensor gather_reduce_rows(const torch::Tensor& src, const torch::Tensor& pos, c10::optional<torch::Tensor> w,
                                 c10::optional<torch::Tensor> out) {
    DXG_CHECK(src.is_cuda() && src.dim() == 2 && src.is_contiguous() && src.scalar_type() == torch::kBFloat16, "src must be contiguous bf16 [M,H]");
    DXG_CHECK(pos.scalar_type() == torch::kInt32 && pos.is_contiguous() && pos.dim() == 2 && pos.size(1) <= 32, "pos must be int32 [N,K], K <= 32");
    const int64_t N = pos.size(0), K = pos.size(1), H = src.size(1);
    DXG_CHECK(H % 8 == 0, "hidden must be a multiple of 8");
    c10::cuda::CUDAGuard guard(src.device());
    torch::Tensor dst = out.has_value() ? *out : torch::empty({N, H}, src.options());
    DXG_CHECK(dst.is_contiguous() && dst.scalar_type() == torch::kBFloat16 && dst.size(0) == N && dst.size(1) == H, "out has the wrong shape");
    const float* wp = nullptr;
    if (w.has_value()) {
        DXG_CHECK(w->scalar_type() == torch::kFloat32 && w->is_contiguous() && w->numel() == N * K, "w must be f32 [N,K]");
        wp = w->data_ptr<float>();
    }
    const cudaError_t e = dx::launch_gather_reduce_rows(src.data_ptr(), dst.data_ptr(), pos.data_ptr<int>(), wp, (int)N, (int)K, (int)H,
                                                        at::cuda::getCurrentCUDAStream(src.device().index()).stream());
    if (e != cudaSuccess) throw std::runtime_error(std::string("gather_reduce_rows: ") + cudaGetErrorString(e));
    return dst;
}

int gemm_error(int device) { return error_flag(device).item<int>(); }
void gemm_clear_error(int device) { error_flag(device).zero_(); }

}  // namespace

torch::Tensor transpose_bf16(const torch::Tensor& x) {
    DXG_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == torch::kBFloat16 && (x.dim() == 2 || x.dim() == 3), "transpose_bf16: contiguous CUDA bf16 [R,C] or [B,R,C]");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.dim() == 3 ? x.size(0) : 1, R = x.size(-2), C = x.size(-1);
    auto out = x.dim() == 3 ? torch::empty({B, C, R}, x.options()) : torch::empty({C, R}, x.options());
    const cudaError_t e = dx::launch_transpose_bf16(x.data_ptr(), out.data_ptr(), (int)B, (int)R, (int)C, at::cuda::getCurrentCUDAStream(x.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "transpose_bf16: rows and cols must be multiples of 8");
    return out;
}

torch::Tensor swiglu_fwd(const torch::Tensor& h13) {
    DXG_CHECK(h13.is_cuda() && h13.is_contiguous() && h13.scalar_type() == torch::kBFloat16 && h13.dim() == 2 && h13.size(1) % 16 == 0, "swiglu_fwd: contiguous CUDA bf16 [M, 2*I], I % 8 == 0");
    c10::cuda::CUDAGuard guard(h13.device());
    const int inter = (int)(h13.size(1) / 2);
    auto h = torch::empty({h13.size(0), inter}, h13.options());
    const cudaError_t e = dx::launch_swiglu_fwd(h13.data_ptr(), h.data_ptr(), h13.size(0), inter, at::cuda::getCurrentCUDAStream(h13.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "swiglu_fwd launch failed");
    return h;
}

torch::Tensor swiglu_bwd(const torch::Tensor& h13, const torch::Tensor& dh) {
    DXG_CHECK(h13.is_cuda() && h13.is_contiguous() && h13.scalar_type() == torch::kBFloat16 && h13.dim() == 2 && h13.size(1) % 16 == 0, "swiglu_bwd: contiguous CUDA bf16 [M, 2*I]");
    DXG_CHECK(dh.is_cuda() && dh.is_contiguous() && dh.scalar_type() == torch::kBFloat16 && dh.dim() == 2 && dh.size(0) == h13.size(0) && dh.size(1) * 2 == h13.size(1), "swiglu_bwd: dh must be bf16 [M, I]");
    c10::cuda::CUDAGuard guard(h13.device());
    auto out = torch::empty_like(h13);
    const cudaError_t e = dx::launch_swiglu_bwd(h13.data_ptr(), dh.data_ptr(), out.data_ptr(), h13.size(0), (int)dh.size(1), at::cuda::getCurrentCUDAStream(h13.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "swiglu_bwd launch failed");
    return out;
}

torch::Tensor rowdot(const torch::Tensor& a, const torch::Tensor& b, const torch::Tensor& pos) {
    DXG_CHECK(a.is_cuda() && a.is_contiguous() && a.scalar_type() == torch::kBFloat16 && a.dim() == 2, "rowdot: a must be contiguous CUDA bf16 [M,H]");
    DXG_CHECK(b.is_cuda() && b.is_contiguous() && b.scalar_type() == torch::kBFloat16 && b.dim() == 2 && b.size(1) == a.size(1), "rowdot: b must be bf16 [N,H]");
    DXG_CHECK(pos.is_cuda() && pos.is_contiguous() && pos.scalar_type() == torch::kInt32 && pos.dim() == 2 && pos.size(0) == b.size(0), "rowdot: pos must be int32 [N,K]");
    c10::cuda::CUDAGuard guard(a.device());
    auto out = torch::empty({pos.size(0), pos.size(1)}, a.options().dtype(torch::kFloat32));
    const cudaError_t e = dx::launch_rowdot(a.data_ptr(), b.data_ptr(), pos.data_ptr<int>(), out.data_ptr<float>(), (int)pos.size(0), (int)pos.size(1), (int)a.size(1),
                                            at::cuda::getCurrentCUDAStream(a.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "rowdot: hidden must be a multiple of 8");
    return out;
}

torch::Tensor build_sf_atoms_a(const torch::Tensor& scales) {
    DXG_CHECK(scales.is_cuda() && scales.scalar_type() == torch::kFloat32 && scales.is_contiguous() && scales.dim() == 2, "scales must be contiguous CUDA f32 [M, K/128]");
    c10::cuda::CUDAGuard guard(scales.device());
    const int64_t M = scales.size(0), nkb = scales.size(1);
    auto atoms = torch::empty({(M + 127) / 128, nkb, 512}, scales.options().dtype(torch::kUInt8));
    const cudaError_t e = dx::launch_build_sfa_atoms(scales.data_ptr<float>(), atoms.data_ptr<uint8_t>(), (int)M, (int)nkb,
                                                     at::cuda::getCurrentCUDAStream(scales.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "build_sf_atoms_a launch failed");
    return atoms;
}

torch::Tensor build_sf_atoms_b(const torch::Tensor& scales, int64_t n, bool swiglu, bool wide) {
    DXG_CHECK(scales.is_cuda() && scales.scalar_type() == torch::kFloat32 && scales.is_contiguous() && scales.dim() == 3 && scales.size(1) * 128 == n,
              "scales must be contiguous CUDA f32 [G, N/128, K/128]");
    c10::cuda::CUDAGuard guard(scales.device());
    const int64_t G = scales.size(0), nkb = scales.size(2);
    DXG_CHECK(!swiglu || (n / 2) % 128 == 0, "build_sf_atoms_b: swiglu needs N/2 % 128 == 0");
    DXG_CHECK(swiglu || !wide || n % 256 == 0, "build_sf_atoms_b: 256-column tiles need N % 256 == 0");
    const int64_t tiles = swiglu ? (wide ? (n / 2) / 128 : (n / 2) / 64) : (wide ? n / 256 : n / 128);
    auto atoms = torch::empty({G, tiles, nkb, wide ? 1024 : 512}, scales.options().dtype(torch::kUInt8));
    const cudaError_t e = dx::launch_build_sfb_atoms(scales.data_ptr<float>(), atoms.data_ptr<uint8_t>(), (int)G, (int)n, (int)nkb, swiglu ? 1 : 0, wide ? 1 : 0,
                                                     at::cuda::getCurrentCUDAStream(scales.get_device()).stream());
    DXG_CHECK(e == cudaSuccess, "build_sf_atoms_b: N (and N/2 with swiglu) must be a multiple of 128");
    return atoms;
}

void bind_gemm(py::module_& m) {
    m.def("build_sf_atoms_a", &build_sf_atoms_a);
    m.def("build_sf_atoms_b", &build_sf_atoms_b, py::arg("scales"), py::arg("n"), py::arg("swiglu") = false, py::arg("wide") = false);
    m.def("transpose_bf16", &transpose_bf16);
    m.def("swiglu_fwd", &swiglu_fwd);
    m.def("swiglu_bwd", &swiglu_bwd);
    m.def("rowdot", &rowdot);
    m.def("grouped_gemm", &grouped_gemm, py::arg("a"), py::arg("b"), py::arg("m_offsets"), py::arg("mode") = 0, py::arg("swiglu") = false,
          py::arg("a_scales") = py::none(), py::arg("b_scales") = py::none(), py::arg("out") = py::none(), py::arg("num_sms") = 0,
          py::arg("timeout_ms") = 2000.0, py::arg("m_ends") = py::none(), py::arg("sfa_atoms") = py::none(), py::arg("sfb_atoms") = py::none(),
          py::arg("ready") = py::none(), py::arg("expected") = py::none(), py::arg("row_info") = py::none(),
          py::arg("scatter_bases") = py::none(), py::arg("trace") = py::none(), py::arg("mn_major") = false,
          py::arg("out_fp8") = py::none(), py::arg("out_atoms") = py::none());
    m.def("build_plan", &build_plan);
    m.def("gather_rows", &gather_rows, py::arg("src"), py::arg("src_row"), py::arg("scale") = py::none(), py::arg("out") = py::none());
    m.def("gather_reduce_rows", &gather_reduce_rows, py::arg("src"), py::arg("pos"), py::arg("w") = py::none(), py::arg("out") = py::none());
    m.def("gemm_error", &gemm_error);
    m.def("gemm_clear_error", &gemm_clear_error);
}
