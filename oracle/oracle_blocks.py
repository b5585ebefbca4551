"""CPU oracle for the two blocks of the hybrid (Mamba-2 + MoE) configuration that the reference does
not contain: the packed-expert ternary MoE layer and the Mamba-2 selective-state-update decode
step.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED BY THE REFERENCE: there is no reference code, test or fixture for these blocks.
The definitions below follow the configuration text (8 experts, top-2 softmax router in fp32,
squared-ReLU experts; 80 heads x 64, d_state 128, one group, conv width 4) and the public Mamba-2
decode-step formulation.  What IS pinned is every ternary product inside them: they go through the
same oracle kernels (``oracle.Kernels``) that are checked bit-for-bit against the reference's
compiled ``matmul_lut_avx512_m1`` / quantiser / RMSNorm.
"""
from __future__ import annotations

import numpy as np

F = np.float32


def silu(v: np.ndarray) -> np.ndarray:
    v = v.astype(F, copy=False)
    return (v / (np.exp(-v) + F(1.0))).astype(F)


def softplus(v: np.ndarray) -> np.ndarray:
    v = v.astype(F, copy=False)
    return np.where(v > F(20.0), v, np.log1p(np.exp(np.minimum(v, F(20.0))))).astype(F)


def moe_route(kern, layer, x: np.ndarray, eps: float):
    """Normalise, route and quantise one token: returns (h_q8, h_scale, experts[2], weights[2]).
    Router: fp32 logits = Wr @ h, softmax over the experts, two largest probabilities (ties to the
    lower index), renormalised to sum to one."""
    H = x.shape[0]
    h = kern.rmsnorm_into(np.ascontiguousarray(x, dtype=F), layer.norm, np.empty(H, F), eps)
    logits = (layer.router.astype(F) @ h).astype(F)
    e = np.exp(logits - logits.max())
    p = (e / e.sum()).astype(F)
    order = sorted(range(p.shape[0]), key=lambda i: (-float(p[i]), i))[:2]
    w = np.array([p[order[0]], p[order[1]]], dtype=F)
    w = (w / (w[0] + w[1])).astype(F)
    q8 = np.empty(H, np.int8)
    s = kern.quantize_activation(h, q8)
    return q8, s, order, w


def moe_layer_step(kern, layer, x: np.ndarray, eps: float, trace: dict = None) -> np.ndarray:
    """x + sum_e w_e * down_e(SubLN(relu2(gate_e h) * up_e h)) for the two routed experts."""
    H = x.shape[0]
    I = layer.intermediate_size
    q8, s, experts, w = moe_route(kern, layer, x, eps)
    ys = []
    for e in experts:
        g = kern.matmul_packed_m1(q8, layer.gate(e), F(layer.scales[e, 0]), s)
        u = kern.matmul_packed_m1(q8, layer.up(e), F(layer.scales[e, 1]), s)
        inter = kern.relu2_mul_into(g, u, np.empty(I, F))
        q2 = np.empty(I, np.int8)
        s2 = kern.rmsnorm_quantize_into(inter, np.ascontiguousarray(layer.sub_norm[e]), q2, np.empty(I, F), eps)
        ys.append(kern.matmul_packed_m1(q2, layer.down(e), F(layer.scales[e, 2]), s2))
    y = (w[0] * ys[0]).astype(F) + (w[1] * ys[1]).astype(F)
    if trace is not None:
        trace.update(experts=experts, weights=w)
    return (x.astype(F) + y).astype(F)


class MambaState:
    """Per-sequence recurrent state of one Mamba-2 layer: the last three conv inputs and the SSM state."""

    def __init__(self, layer):
        self.conv = np.zeros((layer.conv_dim, 3), F)            # oldest .. newest
        self.ssm = np.zeros((layer.nheads, layer.headdim, layer.d_state), F)


def mamba_layer_step(kern, layer, st: MambaState, x: np.ndarray, eps: float) -> np.ndarray:
    """One decode step of a Mamba-2 layer (ngroups = 1):
         zxbcdt = in_proj(quant(RMSNorm(x)));  z | xBC | dt = split
         xBC    = SiLU(conv1d_step(xBC) + bias)            (depthwise, width 4, state = last 3 inputs)
         dt     = softplus(dt + dt_bias);  dA = exp(dt * A)
         state  = state * dA + (dt * x) (outer) B;   y = state . C + D * x
         out    = out_proj(quant(RMSNorm(y * SiLU(z))));  return x + out
    """
    H = x.shape[0]
    di, N, nh, P = layer.d_inner, layer.d_state, layer.nheads, layer.headdim
    q8 = np.empty(H, np.int8)
    s = kern.rmsnorm_quantize_into(np.ascontiguousarray(x, dtype=F), layer.norm, q8, np.empty(H, F), eps)
    zx = kern.matmul_packed_m1(q8, layer.in_proj.w_packed, F(layer.in_proj.scale), s)
    z, xbc_raw, dt_raw = zx[:di], zx[di:di + layer.conv_dim], zx[di + layer.conv_dim:]
    w, b = layer.conv_w, layer.conv_b
    acc = b.astype(F)
    for j in range(3):
        acc = (acc + (w[:, j] * st.conv[:, j]).astype(F)).astype(F)
    acc = (acc + (w[:, 3] * xbc_raw).astype(F)).astype(F)
    st.conv[:, 0:2] = st.conv[:, 1:3]
    st.conv[:, 2] = xbc_raw
    xbc = silu(acc)
    xs = xbc[:di].reshape(nh, P)
    B = xbc[di:di + N]
    C = xbc[di + N:di + 2 * N]
    dt = softplus((dt_raw + layer.dt_bias).astype(F))
    dA = np.exp((dt * layer.A).astype(F)).astype(F)
    dtx = (dt[:, None] * xs).astype(F)
    st.ssm = (st.ssm * dA[:, None, None] + dtx[:, :, None] * B[None, None, :]).astype(F)
    y = ((st.ssm * C[None, None, :]).sum(axis=-1, dtype=F) + layer.D[:, None] * xs).astype(F).reshape(di)
    v = (y * silu(z)).astype(F)
    q2 = np.empty(di, np.int8)
    s2 = kern.rmsnorm_quantize_into(np.ascontiguousarray(v), layer.gated_norm, q2, np.empty(di, F), eps)
    out = kern.matmul_packed_m1(q2, layer.out_proj.w_packed, F(layer.out_proj.scale), s2)
    return (x.astype(F) + out).astype(F)


class HybridState:
    def __init__(self, model):
        self.layers = [MambaState(L) if L.kind == "mamba" else None for L in model.layers]


def hybrid_forward_one(kern, oracle_mod, model, st: HybridState, token_id: int) -> np.ndarray:
    """Embedding -> alternating Mamba-2 / MoE layers -> final RMSNorm -> tied bf16 LM head."""
    eps = model.config.rms_norm_eps
    x = oracle_mod.bf16_to_f32(model.embed_tokens[token_id:token_id + 1])[0].copy()
    for L, ls in zip(model.layers, st.layers):
        x = mamba_layer_step(kern, L, ls, x, eps) if L.kind == "mamba" else moe_layer_step(kern, L, x, eps)
    h = kern.rmsnorm_into(x, model.final_norm, np.empty(x.shape[0], F), eps)
    return kern.lm_head_bf16(model.embed_tokens, h, np.empty(model.config.vocab_size, F))


def hybrid_generate(kern, oracle_mod, model, prompt, max_new_tokens: int):
    """Greedy decode; the prompt is consumed one token at a time (the recurrence is sequential)."""
    st = HybridState(model)
    logits = None
    for t in prompt:
        logits = hybrid_forward_one(kern, oracle_mod, model, st, int(t))
    out = []
    for _ in range(max_new_tokens):
        nxt = int(np.argmax(logits))
        out.append(nxt)
        if len(out) == max_new_tokens:
            break
        logits = hybrid_forward_one(kern, oracle_mod, model, st, nxt)
    return out
