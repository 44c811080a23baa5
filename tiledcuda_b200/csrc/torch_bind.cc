// torch.ops.tiledcuda.*: the reference's operator registry (src/torch_bind.cc:8-11 registers scatter_nd
// and flash_attention_fwd) re-created over the C ABI, plus the ops the reference only has as C++
// examples (gemm, back2back_gemm) or names without code (lstm_cell). Every op writes into
// caller-allocated tensors and returns nothing, launches on the current CUDA stream and never
// synchronises. A failing status becomes a c10::Error (RuntimeError in Python); there is no CPU
// kernel registered, so a CPU tensor is a dispatcher error, not a fallback.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <initializer_list>
#include <vector>

#include "../../include/tiledcuda_b200.h"

namespace {

void check(const char* op, int status) {
    TORCH_CHECK(status == TC_OK, "tiledcuda::", op, " failed with status ", status, ": ", tc_last_error());
}

tc_stream_t stream_of(const at::Tensor& t) {
    return static_cast<tc_stream_t>(c10::cuda::getCurrentCUDAStream(t.get_device()).stream());
}

void need(const at::Tensor& t, const char* name, at::ScalarType dtype) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.scalar_type() == dtype, name, " must be ", dtype, ", got ", t.scalar_type());
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

// Every tensor of a call lives on the device of the first one: the C ABI takes raw pointers and cannot tell.
void same_device(const char* op, const at::Tensor& first, std::initializer_list<const at::Tensor*> rest) {
    for (const at::Tensor* t : rest)
        TORCH_CHECK(t->device() == first.device(), op, ": all tensors must be on one device (got ", first.device(), " and ",
                    t->device(), ")");
}

// Shape rules shared by both scatter ops: indices [..., k] with k <= data.dim(), and updates holding exactly one
// slice (the trailing data.dim() - k dimensions of data) per index tuple. Returns n, the number of tuples.
int64_t scatter_shapes(const char* op, const at::Tensor& data, const at::Tensor& updates, const at::Tensor& indices) {
    TORCH_CHECK(data.is_cuda() && updates.is_cuda() && indices.is_cuda(), op, " needs CUDA tensors");
    same_device(op, data, {&updates, &indices});
    TORCH_CHECK(data.is_contiguous() && updates.is_contiguous() && indices.is_contiguous(), op, " needs contiguous tensors");
    TORCH_CHECK(updates.scalar_type() == data.scalar_type(), op, ": updates and data must have the same dtype");
    TORCH_CHECK(indices.scalar_type() == at::kLong || indices.scalar_type() == at::kInt, op, ": indices must be int32 or int64");
    TORCH_CHECK(indices.dim() >= 1 && data.dim() >= 1, op, ": indices and data must have at least one dimension");
    const int64_t k = indices.size(-1);
    TORCH_CHECK(k >= 1 && k <= data.dim(), op, ": index tuples of length ", k, " do not fit a table of rank ", data.dim());
    const int64_t n = indices.numel() / k;
    int64_t slice = 1;
    for (int64_t i = k; i < data.dim(); ++i) slice *= data.size(i);
    TORCH_CHECK(updates.numel() == n * slice, op, ": updates has ", updates.numel(), " elements, ", n, " tuples of ", slice,
                " elements need ", n * slice);
    return n;
}

// Same argument order as the reference's custom_scatter_op(data, updates, indices)
// (include/kernels/scatter_nd.hpp:39-40). data keeps its N-D shape; indices is [..., k].
void scatter_nd_op(at::Tensor& data, const at::Tensor& updates, const at::Tensor& indices) {
    const int64_t n = scatter_shapes("scatter_nd", data, updates, indices);
    const bool i64 = indices.scalar_type() == at::kLong;
    const int64_t k = indices.size(-1);
    std::vector<int64_t> dims(data.sizes().begin(), data.sizes().end());
    c10::cuda::CUDAGuard guard(data.device());
    check("scatter_nd", tc_scatter_nd(data.data_ptr(), updates.data_ptr(), indices.data_ptr(), i64 ? 1 : 0, dims.data(),
                                      static_cast<int>(dims.size()), n, static_cast<int>(k),
                                      static_cast<int>(data.element_size()), stream_of(data)));
}

// The accumulating form, which is what the reference's kernel does (src/kernels/scatter_nd.cu:44-47).
void scatter_nd_add_op(at::Tensor& data, const at::Tensor& updates, const at::Tensor& indices) {
    const int64_t n = scatter_shapes("scatter_nd_add", data, updates, indices);
    int elem_type = -1;
    switch (data.scalar_type()) {
        case at::kFloat: elem_type = 0; break;
        case at::kHalf: elem_type = 1; break;
        case at::kInt: elem_type = 2; break;
        case at::kDouble: elem_type = 3; break;
        default: TORCH_CHECK(false, "scatter_nd_add supports float32, float16, int32 and float64 tables");
    }
    const bool i64 = indices.scalar_type() == at::kLong;
    const int64_t k = indices.size(-1);
    std::vector<int64_t> dims(data.sizes().begin(), data.sizes().end());
    c10::cuda::CUDAGuard guard(data.device());
    check("scatter_nd_add", tc_scatter_nd_add(data.data_ptr(), updates.data_ptr(), indices.data_ptr(), i64 ? 1 : 0, dims.data(),
                                              static_cast<int>(dims.size()), n, static_cast<int>(k), elem_type, stream_of(data)));
}

// Same signature as custom_flash_attention_op (include/kernels/flash_attn.hpp:35-37): flattened fp16
// Q [m,k], K [n,k], V^T [p,n], O [m,p]; one head; no softmax scale.
void flash_attention_fwd_op(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O, int64_t m,
                            int64_t n, int64_t k, int64_t p) {
    need(Q, "Q", at::kHalf);
    need(K, "K", at::kHalf);
    need(V, "V", at::kHalf);
    need(O, "O", at::kHalf);
    same_device("flash_attention_fwd", Q, {&K, &V, &O});
    TORCH_CHECK(m > 0 && n > 0 && k > 0 && p > 0, "flash_attention_fwd: m, n, k, p must be positive");
    TORCH_CHECK(Q.numel() == m * k && K.numel() == n * k && V.numel() == n * p && O.numel() == m * p,
                "flash_attention_fwd: tensor sizes do not match m, n, k, p");
    c10::cuda::CUDAGuard guard(Q.device());
    check("flash_attention_fwd", tc_flash_attn_fwd_f16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), nullptr, 1, 1, m,
                                                       n, k, p, 1.0f, 1, stream_of(Q)));
}

// Batched, scaled attention: Q [B,H,Sq,D], K [B,H,Skv,D], V [B,H,Skv,Dv] (or V^T), O [B,H,Sq,Dv].
void flash_attn_op(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O, double scale,
                   bool v_is_transposed) {
    need(Q, "Q", at::kHalf);
    need(K, "K", at::kHalf);
    need(V, "V", at::kHalf);
    need(O, "O", at::kHalf);
    same_device("flash_attn", Q, {&K, &V, &O});
    TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4 && O.dim() == 4, "flash_attn: tensors must be [B,H,S,D]");
    const int64_t b = Q.size(0), h = Q.size(1), sq = Q.size(2), d = Q.size(3), skv = K.size(2);
    const int64_t dv = v_is_transposed ? V.size(2) : V.size(3);
    TORCH_CHECK(K.size(0) == b && K.size(1) == h && K.size(3) == d, "flash_attn: K shape mismatch");
    TORCH_CHECK(V.size(0) == b && V.size(1) == h && (v_is_transposed ? V.size(3) : V.size(2)) == skv, "flash_attn: V shape mismatch");
    TORCH_CHECK(O.size(0) == b && O.size(1) == h && O.size(2) == sq && O.size(3) == dv, "flash_attn: O shape mismatch");
    c10::cuda::CUDAGuard guard(Q.device());
    check("flash_attn", tc_flash_attn_fwd_f16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), nullptr, b, h, sq, skv, d, dv,
                                              static_cast<float>(scale), v_is_transposed ? 1 : 0, stream_of(Q)));
}

// flash_attn with a causal mask (bottom-right aligned) and / or [B,S,H,D] operands.
void flash_attn_ex_op(const at::Tensor& Q, const at::Tensor& K, const at::Tensor& V, at::Tensor& O, double scale, bool causal,
                      bool seq_major) {
    need(Q, "Q", at::kHalf);
    need(K, "K", at::kHalf);
    need(V, "V", at::kHalf);
    need(O, "O", at::kHalf);
    same_device("flash_attn_ex", Q, {&K, &V, &O});
    TORCH_CHECK(Q.dim() == 4 && K.dim() == 4 && V.dim() == 4 && O.dim() == 4, "flash_attn_ex: tensors must be 4-D");
    const int sd = seq_major ? 1 : 2, hd = seq_major ? 2 : 1;
    const int64_t b = Q.size(0), h = Q.size(hd), sq = Q.size(sd), d = Q.size(3), skv = K.size(sd), dv = V.size(3);
    TORCH_CHECK(K.size(0) == b && K.size(hd) == h && K.size(3) == d, "flash_attn_ex: K shape mismatch");
    TORCH_CHECK(V.size(0) == b && V.size(hd) == h && V.size(sd) == skv, "flash_attn_ex: V shape mismatch");
    TORCH_CHECK(K.size(sd) == skv, "flash_attn_ex: K shape mismatch");
    TORCH_CHECK(O.size(0) == b && O.size(hd) == h && O.size(sd) == sq && O.size(3) == dv, "flash_attn_ex: O shape mismatch");
    c10::cuda::CUDAGuard guard(Q.device());
    check("flash_attn_ex", tc_flash_attn_fwd_ex_f16(Q.data_ptr(), K.data_ptr(), V.data_ptr(), O.data_ptr(), nullptr, b, h, sq, skv, d,
                                                    dv, static_cast<float>(scale), 0, causal ? 1 : 0, seq_major ? 1 : 0, stream_of(Q)));
}

// C[M,N] fp32 = A[M,K] @ B[N,K]^T (B is the column-major operand of the reference's GEMM examples).
void gemm_op(const at::Tensor& A, const at::Tensor& B, at::Tensor& C) {
    need(A, "A", at::kHalf);
    need(B, "B", at::kHalf);
    need(C, "C", at::kFloat);
    same_device("gemm", A, {&B, &C});
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && C.dim() == 2, "gemm: tensors must be 2-D");
    TORCH_CHECK(B.size(1) == A.size(1) && C.size(0) == A.size(0) && C.size(1) == B.size(0), "gemm: shape mismatch");
    c10::cuda::CUDAGuard guard(A.device());
    check("gemm", tc_gemm_f16_f32(A.data_ptr(), B.data_ptr(), C.data_ptr(), A.size(0), B.size(0), A.size(1), A.size(1), B.size(1),
                                  C.size(1), stream_of(A)));
}

// E fp32 [.., M,P] = fp16(A @ B^T) @ D^T; A [.., M,K], B [.., N,K], D [.., P,N]; 2-D or batched 3-D.
void back2back_gemm_op(const at::Tensor& A, const at::Tensor& B, const at::Tensor& D, at::Tensor& E) {
    need(A, "A", at::kHalf);
    need(B, "B", at::kHalf);
    need(D, "D", at::kHalf);
    need(E, "E", at::kFloat);
    same_device("back2back_gemm", A, {&B, &D, &E});
    TORCH_CHECK((A.dim() == 2 || A.dim() == 3) && B.dim() == A.dim() && D.dim() == A.dim() && E.dim() == A.dim(),
                "back2back_gemm: tensors must all be 2-D or all 3-D");
    const int64_t batch = A.dim() == 3 ? A.size(0) : 1;
    const int64_t m = A.size(-2), k = A.size(-1), n = B.size(-2), p = D.size(-2);
    TORCH_CHECK(B.size(-1) == k && D.size(-1) == n && E.size(-2) == m && E.size(-1) == p, "back2back_gemm: shape mismatch");
    TORCH_CHECK(A.dim() == 2 || (B.size(0) == batch && D.size(0) == batch && E.size(0) == batch), "back2back_gemm: batch mismatch");
    c10::cuda::CUDAGuard guard(A.device());
    check("back2back_gemm", tc_b2b_gemm_f16(A.data_ptr(), B.data_ptr(), D.data_ptr(), E.data_ptr(), m, n, k, p, batch, stream_of(A)));
}

// One LSTM cell step, gate order (i, f, g, o); bias may be an undefined tensor (None).
void lstm_cell_op(const at::Tensor& W, const at::Tensor& U, const c10::optional<at::Tensor>& bias, const at::Tensor& x,
                  const at::Tensor& h_prev, const at::Tensor& c_prev, at::Tensor& h_out, at::Tensor& c_out) {
    need(W, "W", at::kHalf);
    need(U, "U", at::kHalf);
    need(x, "x", at::kHalf);
    need(h_prev, "h_prev", at::kHalf);
    need(h_out, "h_out", at::kHalf);
    need(c_prev, "c_prev", at::kFloat);
    need(c_out, "c_out", at::kFloat);
    const float* b = nullptr;
    if (bias.has_value() && bias->defined()) {
        need(*bias, "bias", at::kFloat);
        b = bias->data_ptr<float>();
    }
    same_device("lstm_cell", x, {&W, &U, &h_prev, &c_prev, &h_out, &c_out});
    TORCH_CHECK(W.dim() == 2 && U.dim() == 2 && x.dim() == 2, "lstm_cell: W, U and x must be 2-D");
    const int64_t batch = x.size(0), input = x.size(1), hidden = U.size(1);
    TORCH_CHECK(W.size(0) == 4 * hidden && W.size(1) == input && U.size(0) == 4 * hidden, "lstm_cell: weight shape mismatch");
    for (const at::Tensor* t : std::initializer_list<const at::Tensor*>{&h_prev, &c_prev, &h_out, &c_out})
        TORCH_CHECK(t->dim() == 2 && t->size(0) == batch && t->size(1) == hidden, "lstm_cell: h_prev, c_prev, h_out and c_out must be [",
                    batch, ", ", hidden, "], got ", t->sizes());
    if (b != nullptr) {
        same_device("lstm_cell", x, {&*bias});
        TORCH_CHECK(bias->numel() == 4 * hidden, "lstm_cell: bias must have 4 * hidden = ", 4 * hidden, " elements, got ", bias->numel());
    }
    TORCH_CHECK(h_out.data_ptr() != h_prev.data_ptr(), "lstm_cell: h_out must not alias h_prev");
    c10::cuda::CUDAGuard guard(x.device());
    check("lstm_cell", tc_lstm_cell_f16(W.data_ptr(), U.data_ptr(), b, x.data_ptr(), h_prev.data_ptr(), c_prev.data_ptr<float>(),
                                        h_out.data_ptr(), c_out.data_ptr<float>(), batch, input, hidden, stream_of(x)));
}

}  // namespace

TORCH_LIBRARY(tiledcuda, m) {
    m.def("scatter_nd(Tensor(a!) data, Tensor updates, Tensor indices) -> ()");
    m.def("flash_attention_fwd(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, int m, int n, int k, int p) -> ()");
    m.def("flash_attn(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, float scale, bool v_is_transposed) -> ()");
    m.def("flash_attn_ex(Tensor Q, Tensor K, Tensor V, Tensor(a!) O, float scale, bool causal, bool seq_major) -> ()");
    m.def("scatter_nd_add(Tensor(a!) data, Tensor updates, Tensor indices) -> ()");
    m.def("gemm(Tensor A, Tensor B, Tensor(a!) C) -> ()");
    m.def("back2back_gemm(Tensor A, Tensor B, Tensor D, Tensor(a!) E) -> ()");
    m.def("lstm_cell(Tensor W, Tensor U, Tensor? bias, Tensor x, Tensor h_prev, Tensor c_prev, Tensor(a!) h_out, "
          "Tensor(b!) c_out) -> ()");
}

TORCH_LIBRARY_IMPL(tiledcuda, CUDA, m) {
    m.impl("scatter_nd", &scatter_nd_op);
    m.impl("flash_attention_fwd", &flash_attention_fwd_op);
    m.impl("flash_attn", &flash_attn_op);
    m.impl("flash_attn_ex", &flash_attn_ex_op);
    m.impl("scatter_nd_add", &scatter_nd_add_op);
    m.impl("gemm", &gemm_op);
    m.impl("back2back_gemm", &back2back_gemm_op);
    m.impl("lstm_cell", &lstm_cell_op);
}
