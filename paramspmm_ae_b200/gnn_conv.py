"""GCN / GIN / AGNN layers over the PCSR operators: mirror of the reference's ``gnn_conv.py``.

Same module and autograd-function names, constructor arguments and forward signatures
(gnn_conv.py:13-238 of the reference).  The layer semantics are the reference's:

* GCN   forward  A (H W); backward AG = A G (A itself: the normalised adjacency is symmetric),
        dH = AG W^T, dW = H^T AG.  With REORDER_NARROW_FIRST (off by default) layers that widen
        their input aggregate first instead, (A H) W.
* GIN   forward  (A X) W; backward dW = (A X)^T G, dX = A (G W^T).
* AGNN  forward  X' = X W, e = SDDMM(X', X') * beta, out = SpMM(e, X'); no edge softmax and no
        row normalisation (the reference has none); the gradient w.r.t. beta follows the
        reference's expression (gnn_conv.py:164-172).
"""
from __future__ import annotations

import math

import torch

n_heads = 1


# When a GCN layer widens its input (fan-in < fan-out) the aggregation is cheaper before the
# projection: A (H W) = (A H) W, and the SpMM then runs at the narrower width.  The reference always
# aggregates after the projection (SpCONV/SpCONV.h:43-72), and so does this module by default, so
# that layer outputs and gradients are the reference's up to the summation order inside the SpMM.
# Setting this to True is an opt-in: results then differ from the reference's by fp32
# re-association of the two products (both orders are tested against fp64 algebra), the backward
# keeps A H instead of H, and the operator is looked up under the input width when the caller's
# dictionary has one for it.
REORDER_NARROW_FIRST = False


def _aggregate(P, X):
    out = P.GIN_spmm(X.contiguous())
    return out[: X.shape[0]] if out.shape[0] != X.shape[0] else out  # block layouts pad the row count


class GCNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, H, weight, ParamSpMM):
        ctx.ParamSpMM = ParamSpMM
        ctx.narrow_first = bool(REORDER_NARROW_FIRST and weight.shape[0] < weight.shape[1])
        if ctx.narrow_first:
            AH = _aggregate(ParamSpMM, H)
            ctx.save_for_backward(AH, weight)
            return torch.mm(AH, weight)
        ctx.save_for_backward(H, weight)
        return ParamSpMM.forward(H, weight)

    @staticmethod
    def backward(ctx, d_output):
        P = ctx.ParamSpMM
        d_output = d_output.contiguous()
        if ctx.narrow_first:
            # dW = (A H)^T G with A H kept from the forward; dH = A (G W^T) (A is symmetric),
            # skipped when the layer input needs no gradient (the first layer).
            AH, weight = ctx.saved_tensors
            d_weight = torch.mm(AH.t(), d_output)
            d_input = _aggregate(P, torch.mm(d_output, weight.t())) if ctx.needs_input_grad[0] else None
            return d_input, d_weight, None
        H, weight = ctx.saved_tensors
        if ctx.needs_input_grad[0]:
            d_input, d_weight = P.backward(d_output, H, weight)
        else:  # the first layer: dH = AG W^T is not formed (the reference forms and drops it)
            d_input, d_weight = P.backward(d_output, H, weight, input_grad=False)
        return d_input, d_weight, None


class GINFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, weight, ParamSpMM):
        X_agg = ParamSpMM.GIN_spmm(X)
        ctx.save_for_backward(X_agg, weight)
        ctx.ParamSpMM = ParamSpMM
        return torch.mm(X_agg, weight)

    @staticmethod
    def backward(ctx, d_output):
        X_agg, weight = ctx.saved_tensors
        d_weight = torch.mm(X_agg.t(), d_output)
        d_input = ctx.ParamSpMM.GIN_spmm(torch.mm(d_output, weight.t()).contiguous())
        return d_input, d_weight, None


# Under torch.no_grad() an AGNN layer on a plain or split CSR operator runs as the fused kernel
# (SDDMM -> scale -> SpMM in one pass).  Set to False to always use the three-kernel composition.
FUSE_AGNN_INFERENCE = True

# With gradients enabled the same layers run AGNNFusedFunction: the forward is the fused kernel, and
# the backward recomputes the edge scores inside the kernel instead of reading a saved edge array,
# so a training step writes no per-edge array at all (the reference's composition writes the
# attention values in the forward and the score gradient in the backward, 4 bytes per edge each,
# gnn_conv.py:130-180).  Outputs and gradients are the reference's up to fp32 summation order.
# Set to False to train through the three-kernel composition (AGNNFunction).
FUSE_AGNN_TRAINING = True
FUSED_APPLY_VEC_WIDTH = 0  # floats per lane per load in the backward pass: 0 = the library's choice, 4 or 8


def _can_fuse(P, dim):
    return getattr(P, "vec_size", 1) == 1 and dim % 4 == 0 and dim <= 256


def _is_operator_colidx(P, colIdx):
    """The fused backward weights edges by the operator's own column ids; callers pass them as an
    [nnz, 1] column (GNN.py:224-225).  Checked once per (operator, tensor) pair, not per step."""
    seen = P.__dict__.setdefault("_colidx_checked", {})
    key = (colIdx.data_ptr(), tuple(colIdx.shape))
    if key not in seen:
        flat = colIdx.reshape(-1)
        seen[key] = bool(flat.shape == P.colIdx.shape and flat.dtype == P.colIdx.dtype and torch.equal(flat, P.colIdx))
    return seen[key]


class AGNNFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, X, weights, attention_w, ParamSpMM, colIdx):
        X_prime = torch.mm(X, weights)
        edge = ParamSpMM.AGNN_sddmm(X_prime)
        # [n_edges] for CSR, [n_blocks, V] for block layouts; one attention head
        edge_attentions = (edge * attention_w.reshape(())).contiguous()
        out = ParamSpMM.AGNN_spmm(edge_attentions, X_prime)
        ctx.save_for_backward(X, weights, edge_attentions)
        ctx.colIdx, ctx.ParamSpMM = colIdx, ParamSpMM
        return out

    @staticmethod
    def backward(ctx, d_output):
        P = ctx.ParamSpMM
        X, weights, edge_attentions = ctx.saved_tensors
        d_output = d_output.contiguous()
        d_prime = P.AGNN_spmm(edge_attentions, d_output)
        d_input = torch.mm(d_prime, weights.t())
        d_weights = torch.mm(X.t(), d_prime)
        d_att = P.AGNN_sddmm(d_output)
        if d_att.dim() != 1:
            d_att = d_att.reshape(-1)[P.mask]  # back to CSR entry order
        d_attention_w = torch.mm(d_att[None, :].expand(n_heads, -1), ctx.colIdx.float()).transpose(0, 1)
        return d_input, d_weights, d_attention_w, None, None


class AGNNFusedFunction(torch.autograd.Function):
    """AGNN layer on a CSR / split-CSR operator without edge arrays.

    forward   X' = X W,  out_i = sum_j beta <X'_i, X'_j> X'_j                 (one fused pass)
    backward  D_i = sum_j beta <X'_i, X'_j> G_j   (fused pass, scores recomputed, gradient rows gathered)
              dX = D W^T,  dW = X^T D                                      (gnn_conv.py:157-160)
              d_beta = sum over edges of <G_i, G_j> * colIdx[e]              (gnn_conv.py:163-172: the
              reference multiplies the score gradient by the column-index column it is handed); here
              as sum_i <G_i, T_i> with T = P H, H_j = j * G_j, P the pattern with unit values: one
              SpMM without a value array and a dot product.
    Like the reference's backward, the edge values are treated as constants with respect to X'."""

    @staticmethod
    def forward(ctx, X, weights, attention_w, P, colIdx):
        from . import ops
        Xp = torch.mm(X, weights)
        split = P.target_row is not None
        beta = float(attention_w.detach().reshape(()))
        out = ops.agnn_fused(Xp, Xp, P.rowPtr, P.colIdx, beta, softmax=False, target_row=P.target_row,
                             n_out_rows=Xp.shape[0] if split else None)
        if not split and out.shape[0] != Xp.shape[0]:  # inputs padded beyond the matrix: zero rows, as the SpMM gives
            out = torch.cat([out, out.new_zeros(Xp.shape[0] - out.shape[0], out.shape[1])])
        ctx.save_for_backward(X, weights, Xp)
        ctx.P, ctx.beta, ctx.colIdx = P, beta, colIdx
        return out

    @staticmethod
    def backward(ctx, d_output):
        from . import ops
        X, weights, Xp = ctx.saved_tensors
        P, beta = ctx.P, ctx.beta
        G = d_output.contiguous()
        split = P.target_row is not None
        n_out = G.shape[0] if split else None

        def apply(A, B, V, b):
            o = ops.agnn_fused(A, B, P.rowPtr, P.colIdx, b, softmax=False, target_row=P.target_row,
                               n_out_rows=n_out, V=V, vec_width=FUSED_APPLY_VEC_WIDTH)
            if o.shape[0] != G.shape[0]:
                o = torch.cat([o, o.new_zeros(G.shape[0] - o.shape[0], o.shape[1])])
            return o

        D = apply(Xp, Xp, G, beta)
        d_input = torch.mm(D, weights.t())
        d_weights = torch.mm(X.t(), D)
        d_att = None
        if ctx.needs_input_grad[2]:
            # The reference weights every edge's score gradient by the float value of the column-index
            # column it is handed, i.e. by the edge's column id j: sum_e <G_i, G_j> j = sum_i <G_i, (P H)_i>
            # with H_j = j G_j and P the pattern with unit values.
            H = G * torch.arange(G.shape[0], device=G.device, dtype=G.dtype)[:, None]
            rows = G.shape[0] if split else P.rowPtr.shape[0] - 1
            T = torch.empty(rows, G.shape[1], device=G.device, dtype=G.dtype)
            ops.spmm_into(T, H, P.rowPtr, P.colIdx, None, target_row=P.target_row, n_out_rows=rows)
            d_att = (G[:rows].double() * T.double()).sum().to(G.dtype).reshape(1, 1)
        return d_input, d_weights, d_att, None, None


class _Conv(torch.nn.Module):
    def __init__(self, input_dim, output_dim):
        super().__init__()
        self.weights = torch.nn.Parameter(torch.randn(input_dim, output_dim))
        self.reset_parameters()

    def reset_parameters(self):
        stdv = 1.0 / math.sqrt(self.weights.size(1))
        self.weights.data.uniform_(-stdv, stdv)

    def _operator(self, spmm_dict):
        dim = self.weights.size(1)
        if dim not in spmm_dict:
            raise ValueError("SpMMDecider not support dim: " + str(dim))
        return spmm_dict[dim]


class GCNConv(_Conv):
    def forward(self, H, spmm_dict):
        P = self._operator(spmm_dict)
        if REORDER_NARROW_FIRST and self.weights.size(0) < self.weights.size(1):
            P = spmm_dict.get(self.weights.size(0), P)  # the aggregation runs at the input width
        return GCNFunction.apply(H, self.weights, P)


class GINConv(_Conv):
    def forward(self, X, spmm_dict):
        return GINFunction.apply(X, self.weights, self._operator(spmm_dict))


class AGNNConv(_Conv):
    def __init__(self, input_dim, output_dim):
        super().__init__(input_dim, output_dim)
        self.attention_w = torch.nn.Parameter(torch.randn(1, n_heads))
        self._beta_cache = (None, 0.0)

    def _beta(self):
        """attention_w as a host float for the fused kernel's by-value argument, read back from the
        device only when the parameter has changed since the last call (in-place updates bump the
        tensor's version counter)."""
        key = (self.attention_w.data_ptr(), self.attention_w._version)
        if self._beta_cache[0] != key:
            self._beta_cache = (key, float(self.attention_w.detach().reshape(())))
        return self._beta_cache[1]

    def forward(self, X, spmm_dict, colIdx):
        P = self._operator(spmm_dict)
        if FUSE_AGNN_INFERENCE and not torch.is_grad_enabled() and _can_fuse(P, self.weights.size(1)):
            # No gradient will be asked for: scores, scaling and aggregation in one kernel, without
            # the per-edge array the backward would need.
            from . import ops
            Xp = torch.mm(X, self.weights)
            split = P.target_row is not None
            return ops.agnn_fused(Xp, Xp, P.rowPtr, P.colIdx, self._beta(), softmax=False,
                                  target_row=P.target_row, n_out_rows=P.mtx_nodes if split else None)
        if (FUSE_AGNN_TRAINING and torch.is_grad_enabled() and _can_fuse(P, self.weights.size(1))
                and _is_operator_colidx(P, colIdx)):
            return AGNNFusedFunction.apply(X, self.weights, self.attention_w, P, colIdx)
        return AGNNFunction.apply(X, self.weights, self.attention_w, P, colIdx)
