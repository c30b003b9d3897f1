"""CPU oracle of the expert-parallel MoE feed-forward step (test infrastructure; see oracle/__init__.py).

No reference implementation exists (the reference has no grouped or MoE kernel); per expert the step is the reference's
dense contract (fp32 accumulate, one cast: include/tritonblas/kernels/stages/matrix_view.py:263-301) applied twice:

    h   = x_t @ [gate | up]_e^T            fp32 accumulators
    act = cast(silu(h_gate) * h_up)        activation on the fp32 accumulators, one cast to the data type
    y   = cast(act @ down_e^T)             fp32 accumulate, one cast
    out = cast(sum_k w[t, k] * y_k)        fp32 sum in k order, one cast

Parity unpinned by construction.
"""
import torch


def moe_ffn_ref(x, topk_ids, topk_weights, w1_of, w2_of, tokens=None):
    """Rows `tokens` (default: all) of the MoE output, in fp32 after the last cast.

    x: (T, H); topk_ids / topk_weights: (T, topk); w1_of(e) -> (2F, H) [gate | up], w2_of(e) -> (H, F), any float dtype.
    """
    dt = x.dtype
    x = x.detach().cpu()
    ids = topk_ids.detach().cpu().to(torch.int64)
    wts = topk_weights.detach().cpu().to(torch.float32)
    tokens = list(range(x.shape[0])) if tokens is None else [int(t) for t in tokens]
    topk = ids.shape[1]
    y = {}
    needed = sorted({int(ids[t, j]) for t in tokens for j in range(topk)})
    for e in needed:
        pairs = [(t, j) for t in tokens for j in range(topk) if int(ids[t, j]) == e]
        rows = torch.stack([x[t] for t, _ in pairs]).to(torch.float32)
        w1 = w1_of(e).detach().cpu().to(torch.float32)
        w2 = w2_of(e).detach().cpu().to(torch.float32)
        f = w1.shape[0] // 2
        h = rows @ w1.T
        act = (torch.nn.functional.silu(h[:, :f]) * h[:, f:]).to(dt).to(torch.float32)
        out = (act @ w2.T).to(dt).to(torch.float32)
        for i, key in enumerate(pairs):
            y[key] = out[i]
    res = torch.zeros(len(tokens), x.shape[1], dtype=torch.float32)
    for i, t in enumerate(tokens):
        acc = torch.zeros(x.shape[1], dtype=torch.float32)
        for j in range(topk):
            acc = acc + wts[t, j] * y[(t, j)]
        res[i] = acc.to(dt).to(torch.float32)
    return res
