// PyTorch extension: the host side of the reference's pybind module `causal_conv1d_cuda`
// (csrc/causal_conv1d.cpp:559-563 — causal_conv1d_fwd / _bwd / _update, same argument
// lists) plus causal_conv1d_varlen_states.  It only inspects tensors, fills the C-ABI
// parameter blocks of include/cc1d.h and calls libcc1d.so on the current stream of the
// tensors' device.  No kernels live here and there is no CPU path: a non-CUDA tensor is an
// error.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

#include "cc1d.h"

namespace {

using OptTensor = std::optional<at::Tensor>;

int dtype_code(const at::Tensor &t, const char *what) {
    switch (t.scalar_type()) {
        case at::ScalarType::Float: return CC1D_F32;
        case at::ScalarType::Half: return CC1D_F16;
        case at::ScalarType::BFloat16: return CC1D_BF16;
        default: TORCH_CHECK(false, what, " must be float32, float16 or bfloat16, got ", t.scalar_type());
    }
}

void need_cuda(const at::Tensor &t, const char *what) {
    TORCH_CHECK(t.is_cuda(), what, " must be a CUDA tensor (this build has no CPU path)");
}

void need_shape(const at::Tensor &t, at::IntArrayRef shape, const char *what) {
    TORCH_CHECK(t.sizes() == shape, what, " must have shape ", shape, ", got ", t.sizes());
}

void raise_on(int rc, const char *fn) {
    TORCH_CHECK(rc == CC1D_OK, fn, ": ", cc1d_status_str(rc));
}

struct ConvDims {
    int64_t batch, dim, seqlen, width;
};

ConvDims conv_dims(const at::Tensor &x, const at::Tensor &weight) {
    TORCH_CHECK(x.dim() == 3, "x must be (batch, dim, seqlen)");
    TORCH_CHECK(weight.dim() == 2, "weight must be (dim, width)");
    ConvDims d{x.size(0), x.size(1), x.size(2), weight.size(1)};
    need_shape(weight, {d.dim, d.width}, "weight");
    TORCH_CHECK(d.width >= 2 && d.width <= 4, "causal_conv1d only supports width between 2 and 4");
    return d;
}

const void *bias_ptr(const OptTensor &bias, const at::Tensor &weight, int64_t dim) {
    if (!bias.has_value()) return nullptr;
    const at::Tensor &b = *bias;
    need_cuda(b, "bias");
    TORCH_CHECK(b.scalar_type() == weight.scalar_type(), "bias must have the dtype of weight");
    need_shape(b, {dim}, "bias");
    TORCH_CHECK(b.stride(-1) == 1 || dim <= 1, "bias must be contiguous");
    return b.data_ptr();
}

const int32_t *seq_idx_ptr(const OptTensor &seq_idx, const ConvDims &d) {
    if (!seq_idx.has_value()) return nullptr;
    const at::Tensor &s = *seq_idx;
    need_cuda(s, "seq_idx");
    TORCH_CHECK(s.scalar_type() == at::kInt, "seq_idx must be int32");
    TORCH_CHECK(s.is_contiguous(), "seq_idx must be contiguous");
    need_shape(s, {d.batch, d.seqlen}, "seq_idx");
    return s.data_ptr<int32_t>();
}

// (batch, dim, width-1) state tensor of x's dtype
void check_state(const at::Tensor &t, const at::Tensor &x, const ConvDims &d, const char *what) {
    need_cuda(t, what);
    TORCH_CHECK(t.scalar_type() == x.scalar_type(), what, " must have the dtype of x");
    need_shape(t, {d.batch, d.dim, d.width - 1}, what);
}

bool channel_last(const at::Tensor &x) { return x.stride(1) == 1 && x.stride(2) > 1; }

}  // namespace

void causal_conv1d_fwd(const at::Tensor &x, const at::Tensor &weight, const OptTensor &bias_,
                       const OptTensor &seq_idx_, const OptTensor &initial_states_, at::Tensor &out,
                       OptTensor &final_states_out_, bool silu_activation) {
    need_cuda(x, "x"); need_cuda(weight, "weight"); need_cuda(out, "out");
    const ConvDims d = conv_dims(x, weight);
    need_shape(out, {d.batch, d.dim, d.seqlen}, "out");
    TORCH_CHECK(out.scalar_type() == x.scalar_type(), "out must have the dtype of x");
    TORCH_CHECK(x.stride(2) == 1 || x.stride(1) == 1, "x must be contiguous along seqlen or along dim");

    cc1d_fwd_params p = {};
    p.itype = dtype_code(x, "x"); p.wtype = dtype_code(weight, "weight");
    p.width = (int32_t)d.width; p.silu = silu_activation;
    p.batch = d.batch; p.dim = d.dim; p.seqlen = d.seqlen;
    p.x = x.data_ptr(); p.x_batch_stride = x.stride(0); p.x_c_stride = x.stride(1); p.x_l_stride = x.stride(2);
    p.weight = weight.data_ptr(); p.weight_c_stride = weight.stride(0); p.weight_width_stride = weight.stride(1);
    p.bias = bias_ptr(bias_, weight, d.dim);
    p.out = out.data_ptr(); p.out_batch_stride = out.stride(0); p.out_c_stride = out.stride(1); p.out_l_stride = out.stride(2);
    p.seq_idx = seq_idx_ptr(seq_idx_, d);
    const bool cl = channel_last(x);
    if (seq_idx_.has_value()) TORCH_CHECK(cl, "seq_idx is only supported for channel last layout");
    if (initial_states_.has_value()) {
        TORCH_CHECK(cl, "initial_states is only supported for channel last layout");
        const at::Tensor &s = *initial_states_;
        check_state(s, x, d, "initial_states");
        TORCH_CHECK(s.stride(1) == 1, "initial_states must have stride(1) == 1");
        p.initial_states = s.data_ptr();
        p.initial_states_batch_stride = s.stride(0); p.initial_states_c_stride = s.stride(1); p.initial_states_l_stride = s.stride(2);
    }
    if (final_states_out_.has_value()) {
        TORCH_CHECK(cl, "final_states is only supported for channel last layout");
        at::Tensor &s = *final_states_out_;
        check_state(s, x, d, "final_states_out");
        TORCH_CHECK(s.stride(1) == 1, "final_states_out must have stride(1) == 1");
        p.final_states = s.data_ptr();
        p.final_states_batch_stride = s.stride(0); p.final_states_c_stride = s.stride(1); p.final_states_l_stride = s.stride(2);
    }
    c10::cuda::CUDAGuard guard(x.device());
    raise_on(cc1d_fwd(&p, at::cuda::getCurrentCUDAStream().stream()), "causal_conv1d_fwd");
}

void causal_conv1d_bwd(const at::Tensor &x, const at::Tensor &weight, const OptTensor &bias_, at::Tensor &dout,
                       const OptTensor &seq_idx_, const OptTensor &initial_states_, const OptTensor &dfinal_states_,
                       at::Tensor &dx, at::Tensor &dweight, OptTensor &dbias_, OptTensor &dinitial_states_,
                       bool silu_activation, bool accumulate, const std::vector<int64_t> &peer_ptrs, int64_t peer_rank,
                       int64_t peer_capacity, const OptTensor &peer_status_, int64_t peer_spin_limit, int64_t phase,
                       const OptTensor &workspace_) {
    need_cuda(x, "x"); need_cuda(weight, "weight"); need_cuda(dout, "dout"); need_cuda(dx, "dx"); need_cuda(dweight, "dweight");
    TORCH_CHECK(bias_.has_value() == dbias_.has_value(), "dbias must be given exactly when bias is");
    const ConvDims d = conv_dims(x, weight);
    need_shape(dout, {d.batch, d.dim, d.seqlen}, "dout");
    need_shape(dx, {d.batch, d.dim, d.seqlen}, "dx");
    need_shape(dweight, {d.dim, d.width}, "dweight");
    TORCH_CHECK(dout.scalar_type() == x.scalar_type() && dx.scalar_type() == x.scalar_type(), "dout and dx must have the dtype of x");
    TORCH_CHECK(dweight.scalar_type() == at::kFloat, "dweight must be float32");
    TORCH_CHECK(x.stride(2) == 1 || x.stride(1) == 1, "x must be contiguous along seqlen or along dim");
    const bool cl = channel_last(x);
    // dout normally arrives in x's layout class.  When autograd hands over the other one: a channel-first
    // dout beside a channel-last x is read in place by the 16-bit kernels (no copy) as long as its rows are
    // 16-byte aligned; every other mixed case is brought into x's layout class by one copy, as in the
    // reference (csrc/causal_conv1d.cpp:297-298).
    at::Tensor dout_l = dout;
    if (!cl && dout.stride(2) != 1) dout_l = dout.contiguous();
    const auto to_channel_last = [](const at::Tensor &t) { return t.transpose(-1, -2).contiguous().transpose(-1, -2); };
    bool dout_in_place = false;
    if (cl && dout.stride(1) != 1 && d.dim > 1) {
        dout_in_place = d.seqlen > 1 && dout.stride(2) == 1 && x.scalar_type() != at::kFloat && dout.stride(1) % 8 == 0 &&
                        (d.batch <= 1 || dout.stride(0) % 8 == 0) && reinterpret_cast<uintptr_t>(dout.data_ptr()) % 16 == 0;
        if (!dout_in_place) dout_l = to_channel_last(dout);
    }
    if (!cl) TORCH_CHECK(dx.stride(2) == 1 || d.seqlen <= 1, "dx must be contiguous along seqlen");
    if (cl) TORCH_CHECK(dx.stride(1) == 1 || d.dim <= 1, "dx must be contiguous along dim");

    cc1d_bwd_params p = {};
    p.itype = dtype_code(x, "x"); p.wtype = dtype_code(weight, "weight");
    p.width = (int32_t)d.width; p.silu = silu_activation;
    p.batch = d.batch; p.dim = d.dim; p.seqlen = d.seqlen;
    p.x = x.data_ptr(); p.x_batch_stride = x.stride(0); p.x_c_stride = x.stride(1); p.x_l_stride = x.stride(2);
    p.weight = weight.data_ptr(); p.weight_c_stride = weight.stride(0); p.weight_width_stride = weight.stride(1);
    p.bias = bias_ptr(bias_, weight, d.dim);
    p.dout = dout_l.data_ptr(); p.dout_batch_stride = dout_l.stride(0); p.dout_c_stride = dout_l.stride(1); p.dout_l_stride = dout_l.stride(2);
    p.dx = dx.data_ptr(); p.dx_batch_stride = dx.stride(0); p.dx_c_stride = dx.stride(1); p.dx_l_stride = dx.stride(2);
    p.dweight = dweight.data_ptr<float>(); p.dweight_c_stride = dweight.stride(0); p.dweight_width_stride = dweight.stride(1);
    if (dbias_.has_value()) {
        at::Tensor &db = *dbias_;
        need_cuda(db, "dbias");
        TORCH_CHECK(db.scalar_type() == at::kFloat, "dbias must be float32");
        need_shape(db, {d.dim}, "dbias");
        TORCH_CHECK(db.stride(0) == 1 || d.dim <= 1, "dbias must be contiguous");
        p.dbias = db.data_ptr<float>();
    }
    p.accumulate = accumulate;
    p.seq_idx = seq_idx_ptr(seq_idx_, d);
    if (seq_idx_.has_value()) TORCH_CHECK(cl, "seq_idx only supported for channel last layout");
    if (initial_states_.has_value()) {
        TORCH_CHECK(cl, "initial_states is only supported for channel last layout");
        const at::Tensor &s = *initial_states_;
        check_state(s, x, d, "initial_states");
        TORCH_CHECK(s.stride(1) == 1, "initial_states must have stride(1) == 1");
        p.initial_states = s.data_ptr();
        p.initial_states_batch_stride = s.stride(0); p.initial_states_c_stride = s.stride(1); p.initial_states_l_stride = s.stride(2);
    }
    if (dfinal_states_.has_value()) {
        TORCH_CHECK(cl, "dfinal_states is only supported for channel last layout");
        const at::Tensor &s = *dfinal_states_;
        check_state(s, x, d, "dfinal_states");
        p.dfinal_states = s.data_ptr();
        p.dfinal_states_batch_stride = s.stride(0); p.dfinal_states_c_stride = s.stride(1); p.dfinal_states_l_stride = s.stride(2);
    }
    if (dinitial_states_.has_value()) {
        TORCH_CHECK(cl, "dinitial_states is only supported for channel last layout");
        at::Tensor &s = *dinitial_states_;
        check_state(s, x, d, "dinitial_states");
        TORCH_CHECK(s.stride(1) == 1, "dinitial_states must have stride(1) == 1");
        p.dinitial_states = s.data_ptr();
        p.dinitial_states_batch_stride = s.stride(0); p.dinitial_states_c_stride = s.stride(1); p.dinitial_states_l_stride = s.stride(2);
    }
    c10::cuda::CUDAGuard guard(x.device());
    // scratch for the fixed-order dweight/dbias reduction: the caller's (it must outlive a
    // backward split into phases), else from torch's caching allocator
    TORCH_CHECK(phase >= 0 && phase <= 2, "phase must be 0, 1 or 2");
    TORCH_CHECK(phase == 0 || workspace_.has_value(), "a backward split into phases needs a caller-provided workspace");
    const size_t ws_bytes = cc1d_bwd_workspace_bytes(&p);
    at::Tensor ws;
    if (workspace_.has_value()) {
        ws = *workspace_;
        need_cuda(ws, "workspace");
        TORCH_CHECK(ws.is_contiguous() && (size_t)ws.nbytes() >= ws_bytes, "workspace must be contiguous and hold ",
                    ws_bytes, " bytes");
    } else {
        ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
    }
    p.workspace = ws.data_ptr();
    p.workspace_bytes = (size_t)ws.nbytes();
    p.phase = (int32_t)phase;
    // ranks of a batch-sharded backward: the finishing kernel also sums dweight / dbias over them
    cc1d_peer_group peers = {};
    if (!peer_ptrs.empty()) {
        TORCH_CHECK(peer_ptrs.size() <= CC1D_MAX_PEERS, "at most ", CC1D_MAX_PEERS, " peers");
        TORCH_CHECK(peer_status_.has_value() && peer_status_->is_cuda() && peer_status_->scalar_type() == at::kInt,
                    "peer_status must be an int32 CUDA tensor");
        peers.world = (int32_t)peer_ptrs.size(); peers.rank = (int32_t)peer_rank; peers.capacity = peer_capacity;
        for (size_t r = 0; r < peer_ptrs.size(); ++r) peers.peer_base[r] = reinterpret_cast<void *>(peer_ptrs[r]);
        peers.status = peer_status_->data_ptr<int32_t>();
        TORCH_CHECK(peer_spin_limit >= 0 && peer_spin_limit <= 0xffffffffll, "peer_spin_limit out of range");
        peers.spin_limit = (uint32_t)peer_spin_limit;
        p.peers = &peers;
    }
    int rc = cc1d_bwd(&p, at::cuda::getCurrentCUDAStream().stream());
    if (dout_in_place && (rc == CC1D_ERR_STRIDE || rc == CC1D_ERR_ALIGN)) {
        // the library could not serve this dout where it lies (e.g. no tensor map for its strides): one copy
        dout_l = to_channel_last(dout);
        p.dout = dout_l.data_ptr(); p.dout_batch_stride = dout_l.stride(0); p.dout_c_stride = dout_l.stride(1); p.dout_l_stride = dout_l.stride(2);
        rc = cc1d_bwd(&p, at::cuda::getCurrentCUDAStream().stream());
    }
    raise_on(rc, "causal_conv1d_bwd");
}

void causal_conv1d_update(const at::Tensor &x, const at::Tensor &conv_state, const at::Tensor &weight,
                          const OptTensor &bias_, at::Tensor &out, bool silu_activation,
                          const OptTensor &cache_seqlens_, const OptTensor &conv_state_indices_) {
    need_cuda(x, "x"); need_cuda(conv_state, "conv_state"); need_cuda(weight, "weight"); need_cuda(out, "out");
    const ConvDims d = conv_dims(x, weight);
    TORCH_CHECK(conv_state.dim() == 3, "conv_state must be (batch, dim, state_len)");
    TORCH_CHECK(conv_state.scalar_type() == x.scalar_type(), "conv_state must have the dtype of x");
    const int64_t state_len = conv_state.size(2);
    TORCH_CHECK(state_len >= d.width - 1, "conv_state_len must be >= width - 1");
    need_shape(out, {d.batch, d.dim, d.seqlen}, "out");
    TORCH_CHECK(out.scalar_type() == x.scalar_type(), "out must have the dtype of x");

    cc1d_update_params p = {};
    p.itype = dtype_code(x, "x"); p.wtype = dtype_code(weight, "weight");
    p.width = (int32_t)d.width; p.silu = silu_activation;
    p.batch = d.batch; p.dim = d.dim; p.seqlen = d.seqlen;
    p.x = x.data_ptr(); p.x_batch_stride = x.stride(0); p.x_c_stride = x.stride(1); p.x_l_stride = x.stride(2);
    p.weight = weight.data_ptr(); p.weight_c_stride = weight.stride(0); p.weight_width_stride = weight.stride(1);
    p.bias = bias_ptr(bias_, weight, d.dim);
    p.out = out.data_ptr(); p.out_batch_stride = out.stride(0); p.out_c_stride = out.stride(1); p.out_l_stride = out.stride(2);
    p.conv_state = conv_state.data_ptr(); p.conv_state_len = state_len;
    p.conv_state_batch_stride = conv_state.stride(0); p.conv_state_c_stride = conv_state.stride(1); p.conv_state_l_stride = conv_state.stride(2);
    if (conv_state_indices_.has_value()) {
        const at::Tensor &idx = *conv_state_indices_;
        need_cuda(idx, "conv_state_indices");
        TORCH_CHECK(idx.scalar_type() == at::kInt, "conv_state_indices must be int32");
        need_shape(idx, {d.batch}, "conv_state_indices");
        TORCH_CHECK(idx.stride(0) == 1 || d.batch <= 1, "conv_state_indices must be contiguous");
        need_shape(conv_state, {conv_state.size(0), d.dim, state_len}, "conv_state");
        p.conv_state_indices = idx.data_ptr<int32_t>();
    } else {
        need_shape(conv_state, {d.batch, d.dim, state_len}, "conv_state");
    }
    if (cache_seqlens_.has_value()) {
        const at::Tensor &cs = *cache_seqlens_;
        need_cuda(cs, "cache_seqlens");
        TORCH_CHECK(cs.scalar_type() == at::kInt, "cache_seqlens must be int32");
        need_shape(cs, {d.batch}, "cache_seqlens");
        TORCH_CHECK(cs.stride(-1) == 1 || d.batch <= 1, "cache_seqlens must be contiguous");
        p.cache_seqlens = cs.data_ptr<int32_t>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    raise_on(cc1d_update(&p, at::cuda::getCurrentCUDAStream().stream()), "causal_conv1d_update");
}

// x: (total_tokens, dim); cu_seqlens: (batch + 1,) int32 or int64; states: (batch, dim, state_len)
void causal_conv1d_varlen_states(const at::Tensor &x, const at::Tensor &cu_seqlens, at::Tensor &states) {
    need_cuda(x, "x"); need_cuda(cu_seqlens, "cu_seqlens"); need_cuda(states, "states");
    TORCH_CHECK(x.dim() == 2 && states.dim() == 3 && cu_seqlens.dim() == 1, "expected x (tokens, dim), cu_seqlens (batch+1,), states (batch, dim, state_len)");
    TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt || cu_seqlens.scalar_type() == at::kLong, "cu_seqlens must be int32 or int64");
    TORCH_CHECK(cu_seqlens.is_contiguous(), "cu_seqlens must be contiguous");
    TORCH_CHECK(states.scalar_type() == x.scalar_type(), "states must have the dtype of x");
    const int64_t batch = cu_seqlens.size(0) - 1;
    need_shape(states, {batch, x.size(1), states.size(2)}, "states");
    cc1d_varlen_states_params p = {};
    p.itype = dtype_code(x, "x");
    p.cu_seqlens_is_int64 = cu_seqlens.scalar_type() == at::kLong;
    p.total_tokens = x.size(0); p.dim = x.size(1); p.batch = batch; p.state_len = states.size(2);
    p.x = x.data_ptr(); p.x_l_stride = x.stride(0); p.x_c_stride = x.stride(1);
    p.cu_seqlens = cu_seqlens.data_ptr();
    p.states = states.data_ptr();
    p.states_batch_stride = states.stride(0); p.states_c_stride = states.stride(1); p.states_l_stride = states.stride(2);
    c10::cuda::CUDAGuard guard(x.device());
    raise_on(cc1d_varlen_states(&p, at::cuda::getCurrentCUDAStream().stream()), "causal_conv1d_varlen_states");
}

// Packed variable-length prefill (cc1d_prefill_varlen): x, out (total_tokens, dim) with
// stride(1) == 1; seq_idx (total_tokens,) int32; cu_seqlens (nseq + 1,) int32; conv states
// (rows, dim, state_len) with stride(1) == 1, read as each sequence's left context and/or
// overwritten with its final state.
void causal_conv1d_prefill_varlen(const at::Tensor &x, const at::Tensor &weight, const OptTensor &bias_,
                                  const at::Tensor &seq_idx, const at::Tensor &cu_seqlens,
                                  const OptTensor &initial_states_, const OptTensor &final_states_,
                                  const OptTensor &state_indices_, const OptTensor &has_initial_state_,
                                  at::Tensor &out, bool silu_activation) {
    need_cuda(x, "x"); need_cuda(weight, "weight"); need_cuda(out, "out"); need_cuda(seq_idx, "seq_idx");
    need_cuda(cu_seqlens, "cu_seqlens");
    TORCH_CHECK(x.dim() == 2 && weight.dim() == 2, "expected x (total_tokens, dim) and weight (dim, width)");
    const int64_t total = x.size(0), dim = x.size(1), width = weight.size(1);
    need_shape(weight, {dim, width}, "weight");
    need_shape(out, {total, dim}, "out");
    TORCH_CHECK(out.scalar_type() == x.scalar_type(), "out must have the dtype of x");
    TORCH_CHECK((x.stride(1) == 1 && out.stride(1) == 1) || dim <= 1, "x and out must be contiguous along dim");
    TORCH_CHECK(seq_idx.scalar_type() == at::kInt && seq_idx.is_contiguous() && seq_idx.numel() == total,
                "seq_idx must be a contiguous int32 tensor of total_tokens entries");
    TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.dim() == 1 && cu_seqlens.is_contiguous() &&
                cu_seqlens.size(0) >= 1, "cu_seqlens must be a contiguous int32 tensor (nseq + 1,)");
    const int64_t nseq = cu_seqlens.size(0) - 1;

    cc1d_prefill_varlen_params p = {};
    p.itype = dtype_code(x, "x"); p.wtype = dtype_code(weight, "weight");
    p.width = (int32_t)width; p.silu = silu_activation;
    p.total_tokens = total; p.dim = dim; p.nseq = nseq;
    p.x = x.data_ptr(); p.x_l_stride = x.stride(0);
    p.weight = weight.data_ptr(); p.weight_c_stride = weight.stride(0); p.weight_width_stride = weight.stride(1);
    p.bias = bias_ptr(bias_, weight, dim);
    p.out = out.data_ptr(); p.out_l_stride = out.stride(0);
    p.seq_idx = seq_idx.data_ptr<int32_t>();
    p.cu_seqlens = cu_seqlens.data_ptr<int32_t>();
    auto state = [&](const at::Tensor &t, const char *what) {
        need_cuda(t, what);
        TORCH_CHECK(t.dim() == 3 && t.size(1) == dim, what, " must be (rows, dim, state_len)");
        TORCH_CHECK(t.scalar_type() == x.scalar_type(), what, " must have the dtype of x");
        TORCH_CHECK(t.stride(1) == 1 || dim <= 1, what, " must have stride(1) == 1");
        TORCH_CHECK(state_indices_.has_value() || t.size(0) >= nseq, what, " has fewer rows than there are sequences");
    };
    if (initial_states_.has_value()) {
        const at::Tensor &t = *initial_states_;
        state(t, "initial_states");
        p.state_len = t.size(2);
        p.initial_states = t.data_ptr();
        p.initial_states_batch_stride = t.stride(0); p.initial_states_l_stride = t.stride(2);
    }
    if (final_states_.has_value()) {
        const at::Tensor &t = *final_states_;
        state(t, "final_states");
        TORCH_CHECK(!initial_states_.has_value() || t.size(2) == p.state_len, "initial_states and final_states differ in state_len");
        p.state_len = t.size(2);
        p.final_states = t.data_ptr();
        p.final_states_batch_stride = t.stride(0); p.final_states_l_stride = t.stride(2);
    }
    if (state_indices_.has_value()) {
        const at::Tensor &t = *state_indices_;
        need_cuda(t, "state_indices");
        TORCH_CHECK(t.scalar_type() == at::kInt && t.is_contiguous() && t.numel() == nseq, "state_indices must be a contiguous int32 tensor (nseq,)");
        p.state_indices = t.data_ptr<int32_t>();
    }
    if (has_initial_state_.has_value()) {
        const at::Tensor &t = *has_initial_state_;
        need_cuda(t, "has_initial_state");
        TORCH_CHECK((t.scalar_type() == at::kBool || t.scalar_type() == at::kByte) && t.is_contiguous() && t.numel() == nseq,
                    "has_initial_state must be a contiguous bool tensor (nseq,)");
        p.has_initial_state = reinterpret_cast<const uint8_t *>(t.data_ptr());
    }
    c10::cuda::CUDAGuard guard(x.device());
    raise_on(cc1d_prefill_varlen(&p, at::cuda::getCurrentCUDAStream().stream()), "causal_conv1d_prefill_varlen");
}

// seq_idx (total_tokens,) int32 <- cu_seqlens (nseq + 1,) int32
void seq_idx_from_cu_seqlens(const at::Tensor &cu_seqlens, at::Tensor &seq_idx) {
    need_cuda(cu_seqlens, "cu_seqlens"); need_cuda(seq_idx, "seq_idx");
    TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.dim() == 1 && cu_seqlens.is_contiguous() &&
                cu_seqlens.size(0) >= 1, "cu_seqlens must be a contiguous int32 tensor (nseq + 1,)");
    TORCH_CHECK(seq_idx.scalar_type() == at::kInt && seq_idx.is_contiguous(), "seq_idx must be a contiguous int32 tensor");
    c10::cuda::CUDAGuard guard(seq_idx.device());
    raise_on(cc1d_seq_idx_from_cu_seqlens(cu_seqlens.data_ptr<int32_t>(), cu_seqlens.size(0) - 1, seq_idx.numel(),
                                          seq_idx.data_ptr<int32_t>(), at::cuda::getCurrentCUDAStream().stream()),
             "seq_idx_from_cu_seqlens");
}

// One-shot peer all-reduce of a small fp32 vector (cc1d_peer_allreduce); peer_ptrs[r] is rank r's
// exchange buffer as mapped on this device.
void peer_allreduce(at::Tensor &buf, const std::vector<int64_t> &peer_ptrs, int64_t rank, int64_t epoch, at::Tensor &status,
                    int64_t spin_limit) {
    need_cuda(buf, "buf"); need_cuda(status, "status");
    TORCH_CHECK(buf.scalar_type() == at::kFloat && buf.is_contiguous(), "buf must be a contiguous float32 tensor");
    TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1, "status must be an int32 tensor");
    TORCH_CHECK(peer_ptrs.size() >= 1 && peer_ptrs.size() <= CC1D_MAX_PEERS, "1..", CC1D_MAX_PEERS, " peers");
    cc1d_peer_allreduce_params p = {};
    p.world = (int32_t)peer_ptrs.size(); p.rank = (int32_t)rank; p.epoch = (uint32_t)epoch;
    TORCH_CHECK(spin_limit >= 0 && spin_limit <= 0xffffffffll, "spin_limit out of range");
    p.spin_limit = (uint32_t)spin_limit;
    p.count = buf.numel();
    p.src = buf.data_ptr<float>(); p.dst = buf.data_ptr<float>();
    for (size_t r = 0; r < peer_ptrs.size(); ++r) p.peer_base[r] = reinterpret_cast<void *>(peer_ptrs[r]);
    p.status = status.data_ptr<int32_t>();
    c10::cuda::CUDAGuard guard(buf.device());
    raise_on(cc1d_peer_allreduce(&p, at::cuda::getCurrentCUDAStream().stream()), "peer_allreduce");
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("causal_conv1d_fwd", &causal_conv1d_fwd, "Causal conv1d forward");
    m.def("causal_conv1d_bwd", &causal_conv1d_bwd, "Causal conv1d backward",
          py::arg("x"), py::arg("weight"), py::arg("bias"), py::arg("dout"), py::arg("seq_idx"),
          py::arg("initial_states"), py::arg("dfinal_states"), py::arg("dx"), py::arg("dweight"),
          py::arg("dbias"), py::arg("dinitial_states"), py::arg("silu_activation"),
          py::arg("accumulate") = true, py::arg("peer_ptrs") = std::vector<int64_t>(), py::arg("peer_rank") = 0,
          py::arg("peer_capacity") = 0, py::arg("peer_status") = py::none(), py::arg("peer_spin_limit") = 0,
          py::arg("phase") = 0, py::arg("workspace") = py::none());
    m.def("bwd_workspace_bytes", [](int64_t batch, int64_t dim, int64_t seqlen, int64_t width, int64_t elem_bytes, bool channel_last) {
        cc1d_bwd_params q = {};
        q.itype = elem_bytes == 4 ? CC1D_F32 : CC1D_BF16; q.wtype = CC1D_F32; q.width = (int32_t)width;
        q.batch = batch; q.dim = dim; q.seqlen = seqlen;
        q.x_c_stride = channel_last ? 1 : seqlen; q.x_l_stride = channel_last ? dim : 1;
        return (int64_t)cc1d_bwd_workspace_bytes(&q);
    }, "Bytes of scratch a backward of this shape needs (cc1d_bwd_workspace_bytes)");
    m.def("causal_conv1d_update", &causal_conv1d_update, "Causal conv1d update");
    m.def("causal_conv1d_varlen_states", &causal_conv1d_varlen_states, "Last tokens of each packed sequence -> conv state");
    m.def("causal_conv1d_prefill_varlen", &causal_conv1d_prefill_varlen, "Packed varlen prefill with per-sequence conv states");
    m.def("seq_idx_from_cu_seqlens", &seq_idx_from_cu_seqlens, "seq_idx of every packed token from cu_seqlens");
    m.def("peer_allreduce", &peer_allreduce, "One-shot all-reduce of a small fp32 vector over peer memory",
          py::arg("buf"), py::arg("peer_ptrs"), py::arg("rank"), py::arg("epoch"), py::arg("status"), py::arg("spin_limit") = 0);
    m.def("peer_allreduce_buffer_bytes", [](int64_t world, int64_t count) { return (int64_t)cc1d_peer_allreduce_buffer_bytes((int32_t)world, count); });
    m.def("wait_expired", []() { return cc1d_wait_expired(); }, "Health check: non-zero if a bounded wait in a kernel ran out (synchronises)");
    m.def("abi_version", []() { return cc1d_abi_version(); });
}
