"""The Mizerax design in the engine against the plain implementation (tests/plain_mizerax.py):
each mechanism alone, whole prompts with the residual after every layer run, token-by-token
decoding, portions down to one and two tokens, mixed batches with pages and slots used again,
``bin/trace_run``, greedy generation through the scheduler; plus kernel-level cases whose
inputs make one far key, a page border, the sink or the first token stand out.  Small
configurations that differ from one another in every size and option."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

from conftest import random_tokens, read_folder
import plain_mizerax as pm
import trace_util as tu

DTYPES = ["float32", "bfloat16"]
F64 = torch.float64


def _attn(heads, kv_heads, dim, vdim, scale, q_temp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp:
        mixer["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return mixer


def _moe(ff, experts, top, identity=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


def _model(vocab, width, max_pos, eps, mult, layers, loop=None):
    cfg = {"architecture": "Mizerax", "vocab": vocab, "width": width, "max_positions": max_pos,
           "norm": {"eps": eps}, "layers": [{"type": "attention", "mixer": m, "mlp": f} for m, f in layers]}
    if mult is not None:
        cfg["residual_mult"] = mult
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


# Four layers of which the two in the middle run twice; values wider than keys; three query
# heads a KV head; a temperature that steps every 7 positions; three of 5 + 2 router outputs a
# token; one layer without a feed-forward, one without a shared expert.
MZ_A = _model(211, 96, 400, 1e-5, 0.7, [
    (_attn(6, 2, 16, 24, 0.3, (0.4, 7)), _moe(40, 5, 3, 2, 56)),
    (_attn(3, 3, 8, 8, 0.35, (0.2, 50)), _moe(24, 4, 2, 1, None)),
    (_attn(4, 1, 24, 8, 0.2), None),
    (_attn(2, 2, 32, 40, 0.18, (1.5, 3)), _moe(40, 5, 3, 2, 56)),
], loop=(1, 3, 2))
# The first layer alone runs three times; one head; one expert a token; no experts without
# tensors in one layer (the key left out) and none in another (given as 0); no multiplier in
# the file; sizes that are no multiple of 8 (the grouped products do not take them).
MZ_B = _model(150, 80, 300, 3e-6, None, [
    (_attn(1, 1, 40, 12, 0.15, (0.3, 16)), _moe(20, 3, 1, None, 28)),
    (_attn(5, 5, 16, 16, 0.25), _moe(16, 6, 4, 0, 16)),
    (_attn(8, 2, 8, 24, 0.4, (0.1, 1)), _moe(12, 2, 2, 3, None)),
], loop=(0, 1, 3))
# Head sizes the tensor-core attention kernels take (keys and values alike): 64 on the tcgen05
# kernel with three query heads a KV head, 32 on the mma.sync one, 128 with four query heads a KV
# head; the loop covers the last two layers.
MZ_C = _model(180, 128, 320, 1e-5, 0.6, [
    (_attn(6, 2, 64, 64, 0.11, (0.35, 20)), _moe(32, 4, 2, 1, 48)),
    (_attn(2, 1, 32, 32, 0.2), None),
    (_attn(4, 1, 128, 128, 0.09, (0.5, 9)), _moe(24, 3, 2, 2, None)),
], loop=(1, 3, 2))
# A width that is no multiple of 4 (no 8- or 16-byte rows anywhere), three query heads on one KV
# head, a loop of ONE pass over both layers (the input mix still runs, once), two of 3 + 1 router
# outputs.
MZ_D = _model(131, 50, 270, 2e-6, 1.3, [
    (_attn(3, 1, 20, 12, 0.22, (0.8, 11)), _moe(20, 3, 2, 1, 12)),
    (_attn(2, 2, 10, 30, 0.3), _moe(12, 2, 1, 1, None)),
], loop=(0, 2, 1))
MZ_CONFIGS = {"mz_a": MZ_A, "mz_b": MZ_B, "mz_c": MZ_C, "mz_d": MZ_D}
MZ_SEEDS = {"mz_a": 7, "mz_b": 8, "mz_c": 10, "mz_d": 12}
# one layer each: a mechanism alone, and no loop at all
MZ_ALONE = {
    "attention_only": _model(97, 64, 200, 1e-5, 1.0, [(_attn(4, 2, 16, 16, 0.25, (0.5, 5)), None)]),
    "routed_ff": _model(97, 64, 200, 1e-5, 0.5, [(_attn(2, 2, 8, 8, 0.3), _moe(24, 6, 2, 2, 32))]),
    "looped": _model(97, 48, 200, 1e-6, 0.9, [(_attn(2, 1, 8, 16, 0.3), _moe(16, 3, 2, 1, 8))], loop=(0, 1, 2)),
}


def _router_outputs(ml):
    return ml["router"]["experts"] + (ml["router"].get("identity") or 0)


def _wide_router_margins(cfg, weights):
    """Make every routed layer's choice a matter of the token id with margins far beyond
    rounding, so that bfloat16 and float64 choose alike.  Channels 0..E-1 of the embedding hold a
    code (the token's j-th router output gets 4 - j); nothing is ever added to those channels
    (position vectors, both per-channel factors and the loop's matrix leave them as they
    are), so the stream keeps the code; the norm passes them with weight 1 and bias 0; router
    row e reads the channels c with c % outputs == e.  The correction lifts ONE output above
    every score, so it is always chosen, with whatever small weight its score gives it."""
    w = {k: v.clone() for k, v in weights.items()}
    routed = [l["mlp"] for l in cfg["layers"] if l.get("mlp")]
    if not routed:
        return w
    E = max(_router_outputs(ml) for ml in routed)
    W = cfg["width"]
    w["embed"][:, :E] = 0.0
    w["pos"][:, :E] = 0.0
    if "loop.in" in w:
        w["loop.in"][:E, :] = 0.0
        for c in range(E):
            w["loop.in"][c, c] = 1.0
    for i, layer in enumerate(cfg["layers"]):
        w[f"l{i}.ls1"][:E] = 0.0
        if f"l{i}.ls2" in w:
            w[f"l{i}.ls2"][:E] = 0.0
        w[f"l{i}.norm1"][:E] = 1.0
        w[f"l{i}.norm1.b"][:E] = 0.0
        ml = layer.get("mlp")
        if ml:
            n_out = _router_outputs(ml)
            r = w[f"l{i}.mlp.router"]
            r[:, :] = 0.0
            for c in range(E):
                r[c % n_out, c] = 1.0
            corr = torch.zeros(n_out)
            if ml["router"]["top"] > 1:
                corr[(i + 1) % n_out] = 2.0
            w[f"l{i}.mlp.correction"] = corr
    # the code must not drown the logits: the last norm lets little of it through
    w["final.norm"][:E] = 0.05
    w["final.norm.b"][:E] = 0.0
    top_most = max(ml["router"]["top"] for ml in routed)
    for tok in range(cfg["vocab"]):
        for j in range(top_most):
            w["embed"][tok, (tok + j) % E] = 4.0 - j
    assert W > E
    return w


@pytest.fixture(scope="module")
def mz_folders(tmp_path_factory):
    from safetensors.torch import save_file
    from helios_b200.weights import write_model_folder

    out = {}
    base = tmp_path_factory.mktemp("mizerax")
    for name, cfg in {**MZ_CONFIGS, **MZ_ALONE}.items():
        folder = write_model_folder(base / name, cfg, MZ_SEEDS.get(name, 9))
        _cfg, weights = read_folder(folder)
        save_file(_wide_router_margins(cfg, weights), str(folder / "model.safetensors"))
        out[name] = folder
    return out


def _bf16(weights):
    return {k: (v.to(torch.bfloat16).float() if v.dim() >= 2 else v) for k, v in weights.items()}


def _plain(cfg, weights, dtype, requests):
    w = _bf16(weights) if dtype == "bfloat16" else weights
    return {rid: pm.forward(cfg, w, toks)[0] for rid, toks in requests.items()}


def _core(folder, dtype, max_tokens, page_size=16, max_slots=4, graphs=True):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype=dtype)
    return EngineCore(model, page_size=page_size, num_pages=-(-max_tokens // page_size),
                      max_slots=max_slots, poison_cache=float("nan"), use_cuda_graphs=graphs)


def _requests(cfg, lengths, seed):
    return {f"q{i}": random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ====================================================================== without a GPU
def test_configuration_is_read_layer_by_layer_and_faults_name_the_key():
    from helios_b200.config import ConfigError
    from helios_b200.config.registry import resolve_architecture

    arch = resolve_architecture(MZ_A)
    assert arch.name == "Mizerax"
    cfg = arch.parse_config(MZ_A)
    assert (cfg.vocab_size, cfg.width, cfg.max_positions, cfg.residual_mult) == (211, 96, 400, 0.7)
    assert cfg.layers[0].mixer.q_temp.every == 7 and cfg.layers[2].mixer.q_temp is None
    assert cfg.layers[0].mlp.identity == 2 and cfg.layers[1].mlp.shared_ff is None and cfg.layers[2].mlp is None
    assert [i for i, _ in cfg.layer_runs()] == [0, 1, 2, 1, 2, 3]
    assert [b for _, b in cfg.layer_runs()] == [False, True, False, True, False, False]
    b = arch.parse_config(MZ_B)
    assert b.residual_mult == 1.0 and b.layers[0].mlp.identity == 0 and b.layers[1].mlp.identity == 0
    assert [i for i, _ in b.layer_runs()] == [0, 0, 0, 1, 2]
    assert arch.parse_config(MZ_ALONE["attention_only"]).loop is None
    empty = copy.deepcopy(MZ_A)
    empty["loop"] = {"start": 2, "stop": 2, "times": 3}
    assert [i for i, _ in arch.parse_config(empty).layer_runs()] == [0, 1, 2, 3]
    empty["loop"] = {"start": 1, "stop": 3, "times": 0}
    none = arch.parse_config(empty)
    assert [i for i, _ in none.layer_runs()] == [0, 3] and not arch.build_plan(none).stages
    for path, value, word in ((("layers", 0, "type"), "conv_mixer", "type"),
                              (("layers", 1, "mixer", "kv_heads"), 2, "kv_heads"),
                              (("layers", 0, "mlp", "router", "top"), 9, "top"),
                              (("layers", 0, "mlp", "kind"), "dense", "kind"),
                              (("loop", "stop"), 9, "loop"),
                              (("norm",), {}, "eps")):
        bad = copy.deepcopy(MZ_A)
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.parse_config(bad)


def test_plan_names_every_tensor_sizes_its_caches_and_orders_the_runs():
    from helios_b200.cache.manager import bytes_per_page, cache_groups_of
    from helios_b200.config.registry import resolve_architecture
    from helios_b200.weights.loader import expected_tensors

    arch = resolve_architecture(MZ_A)
    plan = arch.build_plan(arch.parse_config(MZ_A))
    names = {k: tuple(v[2].shape) for k, v in expected_tensors(plan).items()}
    assert names["embed"] == (211, 96) and names["pos"] == (400, 96) and names["loop.in"] == (96, 192)
    assert names["final.norm"] == (96,) and names["final.norm.b"] == (96,) and plan.tied == {"head": "embed"}
    assert names["l0.norm1"] == (96,) and names["l0.norm1.b"] == (96,) and names["l0.ls1"] == (96,)
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.k"] == (32, 96) and names["l0.mix.v"] == (48, 96)
    assert names["l0.mix.o"] == (96, 144) and names["l0.mix.g"] == (6, 96) and names["l0.mix.q.norm"] == (16,)
    assert names["l0.mlp.router"] == (7, 96) and names["l0.mlp.correction"] == (7,)
    assert names["l0.mlp.e4.down"] == (96, 40) and "l0.mlp.e5.gate" not in names
    assert names["l0.mlp.shared.up"] == (56, 96) and "l1.mlp.shared.up" not in names
    assert "l2.ls2" not in names and "l2.mlp.router" not in names and "l2.ls1" in names
    # six runs, each with a cache of its own; the loop's stage stands before both passes
    assert [(r.layer, r.before) for r in plan.schedule] == \
        [(0, None), (1, "loop."), (2, None), (1, "loop."), (2, None), (3, None)]
    specs, where = cache_groups_of(plan)
    assert sorted(where) == [0, 1, 2, 3, 4, 5]
    assert [(s.num_kv_heads, s.head_dim, s.value_dim) for s in specs] == \
        [(2, 16, 24), (3, 8, None), (1, 24, 8), (2, 32, 40)]
    assert bytes_per_page(plan, 16, 2) == [1 * 16 * 2 * 40 * 2, 2 * 16 * 3 * 16 * 2, 2 * 16 * 1 * 32 * 2,
                                          1 * 16 * 2 * 72 * 2]
    # a model without a loop has no stage and no tensor for it
    alone = resolve_architecture(MZ_ALONE["attention_only"])
    p1 = alone.build_plan(alone.parse_config(MZ_ALONE["attention_only"]))
    assert "loop.in" not in expected_tensors(p1) and not p1.stages


def test_toy_model_of_the_design_from_the_command_line(tmp_path):
    from helios_b200.cli import main

    out = tmp_path / "toy"
    assert main(["make-toy-model", "--arch", "mizerax", "--out", str(out), "--layers", "4", "--hidden-size", "48",
                 "--heads", "2", "--kv-heads", "1", "--vocab-size", "120", "--max-pos", "64"]) == 0
    cfg, weights = read_folder(out)
    assert cfg["architecture"] == "Mizerax" and cfg["loop"] == {"start": 1, "stop": 3, "times": 2}
    assert "loop.in" in weights and "l0.mlp.correction" in weights and "l3.mlp.router" not in weights
    assert main(["info", "--model", str(out)]) == 0
    logits, _ = pm.forward(cfg, weights, [1, 2, 3])
    assert logits.shape == (3, 120) and torch.isfinite(logits).all()


def test_the_number_of_positions_may_come_from_the_position_table(tmp_path):
    from helios_b200.config.registry import load_config
    from helios_b200.weights import write_model_folder

    folder = write_model_folder(tmp_path / "m", MZ_ALONE["looped"], 3)
    stripped = copy.deepcopy(MZ_ALONE["looped"])
    del stripped["max_positions"]
    with open(folder / "config.json", "w") as f:
        json.dump(stripped, f)
    assert load_config(folder).max_positions == 200


def test_the_plain_model_decodes_as_it_prefills():
    """The oracle itself: a prompt at once against the same tokens fed in three portions."""
    from helios_b200.weights.random_init import random_tensors
    from helios_b200.config.registry import resolve_architecture

    arch = resolve_architecture(MZ_B)
    weights = random_tensors(arch.build_plan(arch.parse_config(MZ_B)), 3)
    toks = random_tokens(MZ_B["vocab"], 23, 1)
    whole, _ = pm.forward(MZ_B, weights, toks)
    past, rows = None, []
    for lo, hi in ((0, 9), (9, 10), (10, 23)):
        lg, new = pm.forward(MZ_B, weights, toks[lo:hi], start=lo, past=past)
        past = new
        rows.append(lg)
    assert (torch.cat(rows) - whole).abs().max() < 1e-9


# ====================================================================== kernels, inputs made to show faults
def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_with_a_pending_sum(dtype):
    """The add of two scaled tensors and the norm in one launch; on chosen rows without
    writing back; the add alone; a width that is no multiple of four."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(1)
    for n, H in ((7, 96), (3, 50), (2, 1030), (5, 2048), (2, 8200)):   # in registers, or through shared memory
        x = torch.randn(n, H, generator=g) * 3 + 1.5
        a, b = torch.randn(n, H, generator=g).to(dt), torch.randn(n, H, generator=g).to(dt)
        sa, sb = torch.rand(H, generator=g) + 0.5, torch.rand(H, generator=g) - 0.5
        w, bias = torch.rand(H, generator=g) + 0.5, torch.randn(H, generator=g)
        new = x.double() + 0.6 * (sa.double() * a.double() + sb.double() * b.double())
        want = pm.layer_norm(new, w.double(), bias.double(), 1e-5)
        tol = 3e-5 if dtype == "float32" else 2e-2
        res = x.cuda().clone()
        out = ops.add_layernorm(res, w.cuda(), bias.cuda(), 1e-5, dt, a=a.cuda(), scale_a=sa.cuda(),
                                b=b.cuda(), scale_b=sb.cuda(), mult=0.6)
        assert (out.double().cpu() - want).abs().max() < tol
        assert (res.double().cpu() - new).abs().max() < 1e-5
        rows = torch.tensor([n - 1, 0], dtype=torch.int32)
        res = x.cuda().clone()
        out = ops.add_layernorm(res, w.cuda(), bias.cuda(), 1e-5, dt, rows=rows.cuda(), a=a.cuda(),
                                scale_a=sa.cuda(), mult=0.6)
        new1 = x.double() + 0.6 * sa.double() * a.double()
        assert (out.double().cpu() - pm.layer_norm(new1, w.double(), bias.double(), 1e-5)[rows.long()]).abs().max() < tol
        assert torch.equal(res.cpu(), x)
        res = x.cuda().clone()
        assert ops.add_layernorm(res, None, None, 0.0, None, a=a.cuda(), b=b.cuda(), scale_b=sb.cuda(), mult=2.0) is None
        assert (res.double().cpu() - (x.double() + 2.0 * (a.double() + sb.double() * b.double()))).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,hd,vd", [("float32", 24, 40), ("bfloat16", 24, 40), ("bfloat16", 64, 32),
                                         ("bfloat16", 128, 128), ("bfloat16", 32, 8), ("float32", 64, 32)])
def test_query_and_key_norm_temperature_and_the_cache_write(dtype, hd, vd):
    """Positions just below, at and above every step of the temperature (every 5: positions 3,
    4, 5, 8, 9, 10) and position 0; keys and values land at the token's place in scrambled
    pages; values of another size than keys; columns behind q | k | v stay as they were."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(2)
    nh, nkv, page, eps, coef, every = 4, 2, 4, 1e-5, 0.7, 5      # heads of 24: one warp a head; 32 to 128: 16-byte pieces
    pos = torch.tensor([0, 3, 4, 5, 8, 9, 10, 14, 15, 33], dtype=torch.int32)
    T = pos.numel()
    ld = nh * hd + nkv * (hd + vd) + 8
    rows = (torch.randn(T, ld, generator=g) * 2).to(dt)
    wq, wk = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5
    order = torch.randperm(12, generator=g).to(torch.int32)
    table = order.view(1, -1).contiguous()
    k_pages = torch.full((13, nkv, page, hd), float("nan"), dtype=dt)
    v_pages = torch.full((13, nkv, page, vd), float("nan"), dtype=dt)
    r = rows.cuda().clone()
    kp, vp = k_pages.cuda(), v_pages.cuda()
    ops.qk_norm_kv_write(r, pos.cuda(), torch.zeros(T, dtype=torch.int32).cuda(), table.cuda(), kp, vp,
                         nh, nkv, hd, vd, page, wq.cuda(), wk.cuda(), eps, coef, every)
    x = rows.double()
    temp = pm.query_temperature(pos.long(), coef, every)
    assert temp[2] == 1.0 + coef * math.log(2.0) and temp[1] == 1.0 and temp[6] == 1.0 + coef * math.log(3.0)
    q = pm.rms_norm(x[:, :nh * hd].view(T, nh, hd), wq.double(), eps) * temp.view(T, 1, 1)
    k = pm.rms_norm(x[:, nh * hd:(nh + nkv) * hd].view(T, nkv, hd), wk.double(), eps)
    tol = 1e-5 if dtype == "float32" else 3e-2
    got = r.double().cpu()
    assert (got[:, :nh * hd].view(T, nh, hd) - q).abs().max() < tol * float(q.abs().max())
    assert torch.equal(got[:, (nh + nkv) * hd:], x[:, (nh + nkv) * hd:])
    for t in range(T):
        p = int(pos[t])
        pg, slot = int(order[p // page]), p % page
        assert (kp[pg, :, slot].double().cpu() - k[t]).abs().max() < tol * float(k.abs().max())
        assert torch.equal(vp[pg, :, slot].double().cpu(), x[t, (nh + nkv) * hd:(nh + nkv) * hd + nkv * vd].view(nkv, vd))
    written = torch.zeros(13, page, dtype=torch.bool)
    for p in pos.tolist():
        written[int(order[p // page]), p % page] = True
    assert torch.isnan(kp.float().cpu()[:, 0][~written]).all()


def _paged(keys, values, page, g, dt):
    """Scatter [n, kvh, d] rows into pages handed out in a scrambled order, NaN elsewhere."""
    n = keys.shape[0]
    n_pages = -(-n // page)
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    kp = torch.full((n_pages + 4, keys.shape[1], page, keys.shape[2]), float("nan"), dtype=dt)
    vp = torch.full((n_pages + 4, values.shape[1], page, values.shape[2]), float("nan"), dtype=dt)
    for j in range(n):
        kp[order[j // page], :, j % page] = keys[j].to(dt)
        vp[order[j // page], :, j % page] = values[j].to(dt)
    return kp, vp, order.to(torch.int32)


def _attend_cases(ops, q, kp, vp, order, q_pos, nh, nkv, hd, vd, page, scale, slopes, sink, gate, max_ctx):
    """Every query is a request of its own with one token, all reading the same pages."""
    from types import SimpleNamespace
    from helios_b200.engine.batch import SeqSlice

    n = q.shape[0]
    dev = "cuda"
    ctx = SimpleNamespace(seq_of_token=torch.arange(n, dtype=torch.int32, device=dev), positions=q_pos.to(dev),
                          start_pos=q_pos.to(dev), context_len=(q_pos + 1).to(dev), extras={}, max_context_len=max_ctx,
                          cu_tokens=torch.arange(n + 1, dtype=torch.int32, device=dev), decode_only=True,
                          max_tokens_per_seq=1, num_tokens=n,
                          seqs=[SeqSlice(None, 0, int(p), 1, i) for i, p in enumerate(q_pos.tolist())], num_seqs=n)
    table = order.view(1, -1).repeat(n, 1).contiguous().to(dev)
    options = ops.AttentionOptions(slopes=None if slopes is None else slopes.float().to(dev), sink=sink,
                                   gate=None if gate is None else gate.to(dev),
                                   value_dim=None if vd == hd else vd)
    return ops.attention(ctx, q.to(dev), kp.to(dev), vp.to(dev), table, nh, nkv, hd, page, None, scale,
                         options=options).float().cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_far_key_page_borders_first_tokens_and_the_sink(dtype):
    """One request of 300 tokens in scrambled pages of 16.  A query is aligned with ONE chosen
    key and scaled so that this key takes nearly all the weight in spite of the distance bias: a
    far key among hundreds, the last key of a page, the first of the next, position 0, the
    query's own position.  Then queries against which every key scores far below 0: the sink
    takes the weight and the output is nearly nothing.  Every case also against the plain
    softmax."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(3)
    n, page, nh, nkv, hd, vd = 300, 16, 4, 2, (40 if dtype == "float32" else 64), (24 if dtype == "float32" else 64)
    keys = torch.randn(n, nkv, hd, generator=g)
    keys[..., -1] = 3.0                     # every key has a positive last channel: a query along -e_last scores all far below 0
    keys = (keys / keys.norm(dim=-1, keepdim=True)).to(dt).float()
    values = torch.randn(n, nkv, vd, generator=g).to(dt).float()
    kp, vp, order = _paged(keys, values, page, g, dt)
    slopes = pm.head_slopes(nh) * 0.2       # the kernel takes any slopes; these take at most 15 off
    cases = [(299, 2), (299, 15), (299, 16), (299, 0), (299, 299), (299, 287), (160, 159), (17, 16),
             (16, 16), (15, 0), (0, 0), (1, 0), (1, 1), (255, 31), (256, 32)]
    q_pos = torch.tensor([c[0] for c in cases] + [299, 40, 0], dtype=torch.int32)
    q = torch.zeros(len(q_pos), nh, hd)
    for i, (p, key) in enumerate(cases):
        for h in range(nh):
            # the chosen key scores 60 after the bias; no other key comes near
            q[i, h] = keys[key, h // (nh // nkv)] * (60.0 + float(slopes[h]) * (p - key))
    for i in range(len(cases), len(q_pos)):
        q[i, :, -1] = -40.0
    q = q.to(dt)
    gate = torch.randn(len(q_pos), nh + 3, generator=g).to(dt)
    out = _attend_cases(ops, q.view(len(q_pos), nh * hd).contiguous(), kp, vp, order, q_pos, nh, nkv, hd, vd, page,
                        1.0, slopes, True, gate.cuda()[:, 1:1 + nh], n).view(len(q_pos), nh, vd)
    rep = nh // nkv
    for i, p in enumerate(q_pos.tolist()):
        kk = keys[:p + 1].double().repeat_interleave(rep, 1)
        vv = values[:p + 1].double().repeat_interleave(rep, 1)
        s = pm.attention_scores(q[i:i + 1].double(), kk, 1.0, slopes)
        w = pm.sink_softmax(s)                                               # [h, 1, keys]
        want = torch.einsum("hij,jhd->ihd", w, vv)[0] * torch.sigmoid(gate[i, 1:1 + nh].double()).unsqueeze(-1)
        tol = 2e-5 if dtype == "float32" else 2e-2
        assert (out[i].double() - want).abs().max() < tol * max(1.0, float(want.abs().max())), (i, p)
        if i < len(cases):
            key = cases[i][1]
            assert float(w[:, 0, key].min()) > 0.99, "the case does not single out its key"
            lone = values[key].double().repeat_interleave(rep, 0) * torch.sigmoid(gate[i, 1:1 + nh].double()).unsqueeze(-1)
            assert (out[i].double() - lone).abs().max() < 0.05 * float(values.abs().max())
    # the sink: every key scores far below 0, the weights add up to next to nothing
    s_last = pm.attention_scores(q[len(cases):len(cases) + 1].double(), keys.double().repeat_interleave(rep, 1), 1.0, slopes)
    assert float(pm.sink_softmax(s_last).sum(-1).max()) < 0.01
    assert float(out[len(cases):].abs().max()) < 0.05
    # ... and without it they do (the kernel's option, not a constant)
    out0 = _attend_cases(ops, q.view(len(q_pos), nh * hd).contiguous(), kp, vp, order, q_pos, nh, nkv, hd, vd, page,
                         1.0, slopes, False, None, n).view(len(q_pos), nh, vd)
    i = len(cases)
    s = pm.attention_scores(q[i:i + 1].double(), keys.double().repeat_interleave(rep, 1), 1.0, slopes)
    want = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), values.double().repeat_interleave(rep, 1))[0]
    assert (out0[i].double() - want).abs().max() < (2e-5 if dtype == "float32" else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,hd,vd", [("float32", 24, 40), ("bfloat16", 64, 64), ("bfloat16", 32, 32),
                                         ("bfloat16", 128, 128), ("bfloat16", 64, 32)])
def test_attention_of_portions_behind_a_prefix_against_the_plain_softmax(dtype, hd, vd):
    """Three requests in one batch: a portion of 37 tokens behind 100 cached ones, a whole
    prompt of 50, one decoded token at position 211; random keys, every row against the plain
    scores with bias, sink and gate.  The sizes take every kernel in turn: one warp a row,
    tcgen05, mma.sync, and one warp a row again where values are smaller than keys."""
    from types import SimpleNamespace
    from helios_b200.csrc import ops
    from helios_b200.engine.batch import SeqSlice

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(5)
    page, nh, nkv = 16, 6, 2
    lens, starts = [137, 50, 212], [100, 0, 211]
    slopes = pm.head_slopes(nh)
    ks = [torch.randn(n, nkv, hd, generator=g).to(dt).float() for n in lens]
    vs = [torch.randn(n, nkv, vd, generator=g).to(dt).float() for n in lens]
    pages_each = [-(-n // page) for n in lens]
    total = sum(pages_each)
    order = torch.randperm(total + 2, generator=g)[:total].to(torch.int32)
    kp = torch.full((total + 3, nkv, page, hd), float("nan"), dtype=dt)
    vp = torch.full((total + 3, nkv, page, vd), float("nan"), dtype=dt)
    table = torch.full((3, max(pages_each)), -1, dtype=torch.int32)
    off = 0
    for r, n in enumerate(lens):
        table[r, :pages_each[r]] = order[off:off + pages_each[r]]
        for j in range(n):
            kp[table[r, j // page], :, j % page] = ks[r][j].to(dt)
            vp[table[r, j // page], :, j % page] = vs[r][j].to(dt)
        off += pages_each[r]
    counts = [lens[r] - starts[r] for r in range(3)]
    T = sum(counts)
    q = (torch.randn(T, nh, hd, generator=g) * 0.7).to(dt)
    gate = torch.randn(T, nh, generator=g).to(dt)
    pos = torch.cat([torch.arange(starts[r], lens[r]) for r in range(3)]).to(torch.int32)
    seq = torch.cat([torch.full((counts[r],), r) for r in range(3)]).to(torch.int32)
    cu = torch.tensor([0, counts[0], counts[0] + counts[1], T], dtype=torch.int32)
    dev = "cuda"
    seqs, o = [], 0
    for r in range(3):
        seqs.append(SeqSlice(None, r, starts[r], counts[r], o))
        o += counts[r]
    ctx = SimpleNamespace(seq_of_token=seq.to(dev), positions=pos.to(dev), start_pos=torch.tensor(starts, dtype=torch.int32, device=dev),
                          context_len=torch.tensor(lens, dtype=torch.int32, device=dev), extras={}, max_context_len=max(lens),
                          cu_tokens=cu.to(dev), decode_only=False, max_tokens_per_seq=max(counts), num_tokens=T,
                          seqs=seqs, num_seqs=3)
    options = ops.AttentionOptions(slopes=slopes.float().to(dev), sink=True, gate=gate.to(dev),
                                   value_dim=None if vd == hd else vd)
    out = ops.attention(ctx, q.view(T, nh * hd).contiguous().to(dev), kp.to(dev), vp.to(dev), table.to(dev), nh, nkv,
                        hd, page, None, 0.21, options=options).float().cpu().view(T, nh, vd)
    rep, o = nh // nkv, 0
    for r in range(3):
        qq = q[o:o + counts[r]].double()
        s = pm.attention_scores(qq, ks[r].double().repeat_interleave(rep, 1), 0.21, slopes)
        want = torch.einsum("hij,jhd->ihd", pm.sink_softmax(s), vs[r].double().repeat_interleave(rep, 1))
        want = want * torch.sigmoid(gate[o:o + counts[r]].double()).unsqueeze(-1)
        tol = 2e-5 if dtype == "float32" else 2e-2
        assert (out[o:o + counts[r]].double() - want).abs().max() < tol, r
        o += counts[r]


@pytest.mark.gpu
@pytest.mark.parametrize("hd,G", [(64, 4), (128, 1), (32, 16), (96, 3)])
def test_decode_kernel_with_its_context_in_one_slice_in_a_cluster_and_merged(hd, G):
    """Five requests of unequal length, one token each, on the split-context decode kernel:
    the context as one slice, as four (merged inside a thread-block cluster) and as twelve
    (merged by a second kernel).  Bias, sink and gate are applied where the slices meet."""
    from helios_b200.csrc import ops

    dt = torch.bfloat16
    g = torch.Generator().manual_seed(8)
    page, nkv = 16, 2
    nh = nkv * G
    lens = [700, 1, 17, 333, 64]
    slopes = pm.head_slopes(nh)
    ks = [torch.randn(n, nkv, hd, generator=g).to(dt).float() for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g).to(dt).float() for n in lens]
    pages_each = [-(-n // page) for n in lens]
    total = sum(pages_each)
    order = torch.randperm(total + 2, generator=g)[:total].to(torch.int32)
    kp = torch.full((total + 3, nkv, page, hd), float("nan"), dtype=dt)
    vp = torch.full((total + 3, nkv, page, hd), float("nan"), dtype=dt)
    table = torch.full((len(lens), max(pages_each)), -1, dtype=torch.int32)
    off = 0
    for r, n in enumerate(lens):
        table[r, :pages_each[r]] = order[off:off + pages_each[r]]
        for j in range(n):
            kp[table[r, j // page], :, j % page] = ks[r][j].to(dt)
            vp[table[r, j // page], :, j % page] = vs[r][j].to(dt)
        off += pages_each[r]
    S = len(lens)
    q = (torch.randn(S, nh, hd, generator=g) * 0.5).to(dt)
    gate = torch.randn(S, nh, generator=g).to(dt)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    options = ops.AttentionOptions(slopes=slopes.float().cuda(), sink=True, gate=gate.cuda())
    want = []
    for r in range(S):
        s = pm.attention_scores(q[r:r + 1].double(), ks[r].double().repeat_interleave(G, 1), 0.17, slopes)
        o = torch.einsum("hij,jhd->ihd", pm.sink_softmax(s), vs[r].double().repeat_interleave(G, 1))
        want.append(o[0] * torch.sigmoid(gate[r].double()).unsqueeze(-1))
    want = torch.stack(want)
    for n_splits in (1, 4, 12):
        out = ops.attention_decode_bf16(q.view(S, nh * hd).contiguous().cuda(), kp.cuda(), vp.cuda(), table.cuda(),
                                        pos.cuda(), nh, nkv, hd, page, None, 0.17, n_splits, options=options)
        assert (out.float().cpu().view(S, nh, hd).double() - want).abs().max() < 2e-2, n_splits


@pytest.mark.gpu
@pytest.mark.parametrize("hd,G,every", [(64, 2, 5), (128, 4, 0), (32, 9, 1), (96, 1, 300)])
def test_decode_kernel_norms_and_writes_on_the_way_in(hd, G, every):
    """The decode kernel given rows straight from the projection (q | k | v | gate) does what
    the launch before it would have done: q and k normed, the temperature on q, the new key
    and value in the pages.  Against that launch followed by the same kernel; positions on
    both sides of a page border and of a step of the temperature."""
    from helios_b200.csrc import ops

    dt = torch.bfloat16
    g = torch.Generator().manual_seed(11)
    page, nkv = 16, 2
    nh = nkv * G
    pos = torch.tensor([0, 15, 16, 4, 5, 299, 300, 47], dtype=torch.int32)
    S = pos.numel()
    pages_each = [int(p) // page + 1 for p in pos]
    total = sum(pages_each)
    order = torch.randperm(total + 2, generator=g)[:total].to(torch.int32)
    kp = (torch.randn(total + 3, nkv, page, hd, generator=g) * 0.5).to(dt)
    vp = torch.randn(total + 3, nkv, page, hd, generator=g).to(dt)
    table = torch.full((S, max(pages_each)), -1, dtype=torch.int32)
    off = 0
    for r in range(S):
        table[r, :pages_each[r]] = order[off:off + pages_each[r]]
        off += pages_each[r]
    ld = (nh + 2 * nkv) * hd + 8 * (-(-nh // 8))
    rows = torch.randn(S, ld, generator=g).to(dt)
    wq, wk = torch.rand(hd, generator=g) + 0.5, torch.rand(hd, generator=g) + 0.5
    slopes = pm.head_slopes(nh).float().cuda()
    seq = torch.arange(S, dtype=torch.int32).cuda()

    def options(r):
        return ops.AttentionOptions(slopes=slopes, sink=True, gate=r[:, (nh + 2 * nkv) * hd:(nh + 2 * nkv) * hd + nh])

    r1, k1, v1 = rows.cuda().clone(), kp.cuda().clone(), vp.cuda().clone()
    ops.qk_norm_kv_write(r1, pos.cuda(), seq, table.cuda(), k1, v1, nh, nkv, hd, hd, page, wq.cuda(), wk.cuda(),
                         1e-5, 0.6, every)
    want = ops.attention_decode_bf16(r1, k1, v1, table.cuda(), pos.cuda(), nh, nkv, hd, page, None, 0.2, 2,
                                     options=options(r1))
    for n_splits in (1, 3):
        r2, k2, v2 = rows.cuda().clone(), kp.cuda().clone(), vp.cuda().clone()
        got = ops.attention_decode_bf16(r2, k2, v2, table.cuda(), pos.cuda(), nh, nkv, hd, page, None, 0.2, n_splits,
                                        write_cache=True, options=options(r2),
                                        qk_norm=(wq.cuda(), wk.cuda(), 1e-5, 0.6, every))
        assert torch.equal(r2.cpu(), rows)                                   # the rows are left as they were
        assert torch.equal(v2.cpu(), v1.cpu())
        assert (k2.float() - k1.float()).abs().max() <= 0.02 * float(k1.float().abs().max())
        assert (got.float() - want.float()).abs().max() < 2e-2 * max(1.0, float(want.float().abs().max()))


@pytest.mark.gpu
@pytest.mark.parametrize("ff", [40, 20])
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_and_experts_against_the_plain_functions(dtype, ff):
    """Same input for both sides: softmax over 5 + 2 router outputs, a correction that changes
    the choice but not the weights, three a token, the weight on the output, experts that return
    their input, an expert for every token.  An inner size of 20 is one the grouped product of the
    bfloat16 path does not take: every pair then streams its expert's rows, as in float32."""
    from helios_b200.csrc import ops

    dt = _dt(dtype)
    dev = "cuda"
    g = torch.Generator().manual_seed(4)
    T, width, E, I, top, shared = 19, 72, 5, 2, 3, 24
    h = torch.randn(T, width, generator=g).to(dt)
    W = {"router": (torch.randn(E + I, width, generator=g) * 0.2).to(dt).float(),
         "correction": torch.tensor([0.0, 0.3, -0.2, 0.0, 0.1, 0.25, -0.1])}
    for e in [f"e{i}." for i in range(E)] + ["shared."]:
        inner = shared if e == "shared." else ff
        W[e + "gate"] = (torch.randn(inner, width, generator=g) * 0.2).to(dt).float()
        W[e + "up"] = (torch.randn(inner, width, generator=g) * 0.2).to(dt).float()
        W[e + "down"] = (torch.randn(width, inner, generator=g) * 0.2).to(dt).float()
    Wd = {k: v.double() for k, v in W.items()}
    ml = {"router": {"experts": E, "identity": I, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared}}
    logits = ops.linear_logits(h.to(dev), W["router"].to(dt).to(dev))
    # both sides choose from the same float32 logits
    s = torch.softmax(logits.double().cpu(), -1)
    _, want_ids = torch.topk(s + Wd["correction"], top, dim=-1)
    want_w = torch.gather(s, -1, want_ids)
    plain_ids, _ = pm.router_choice(h.double(), Wd, "", top)
    assert not torch.equal(torch.topk(s, top, dim=-1).indices, want_ids), "the correction changes nothing here"
    assert (want_ids >= E).any() and torch.equal(plain_ids, want_ids)
    ids, weights = ops.moe_topk(logits, top, "softmax", W["correction"].to(dev))
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (weights.cpu().double() - want_w).abs().max() < 1e-6
    w_gu = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]).to(dt).to(dev)
    w_d = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(dt).to(dev)
    base = ops.linear(ops.linear_swiglu(h.to(dev), torch.cat([W["shared.gate"], W["shared.up"]]).to(dt).to(dev)),
                      W["shared.down"].to(dt).to(dev))
    got = ops.moe_experts(h.to(dev), ids, weights, w_gu, w_d, gate="silu", weight_on="output", identity=I,
                          base=base).float().cpu().double()
    want = pm.routed_ff(h.double(), Wd, "", ml)
    tol = 2e-5 if dtype == "float32" else 3e-2 * float(want.abs().max())
    assert (got - want).abs().max() < tol
    # rows of NaN (the padding of captured steps may bring them) still yield distinct, valid ids;
    # so do rows of equal logits (lower index first) and more router outputs than a warp has lanes
    for n_out in (E + I, 40, 300):
        odd = torch.zeros(3, n_out)
        odd[0] = float("nan")
        odd[2, 7 % n_out] = float("nan")
        for kind in ("softmax", "sigmoid"):
            ids3, _ = ops.moe_topk(odd.to(dev), top, kind)
            ids3 = ids3.cpu().tolist()
            assert all(len(set(r)) == top and all(0 <= e < n_out for e in r) for r in ids3), (n_out, kind, ids3)
            assert ids3[1] == list(range(top))
    # the sigmoid router with a correction too, and the old form (weight on the input) still
    ids2, w2 = ops.moe_topk(logits, 2, "sigmoid", W["correction"].to(dev))
    sg = torch.sigmoid(logits.double().cpu())
    assert torch.equal(ids2.cpu().long(), torch.topk(sg + Wd["correction"], 2, dim=-1).indices)
    assert (w2.cpu().double() - torch.gather(sg, -1, ids2.cpu().long())).abs().max() < 1e-6


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_input_mix(dtype):
    """x <- W [x ; x0] with the stream float32 on both sides."""
    from types import SimpleNamespace
    from helios_b200.parts import StreamInputMix

    dt = _dt(dtype)
    g = torch.Generator().manual_seed(6)
    T, W = 11, 40
    part = StreamInputMix(W, tensor_name="in")
    w = (torch.randn(W, 2 * W, generator=g) * 0.3).to(dt)
    part.bind({"in": w.cuda()})
    x, x0 = torch.randn(T, W, generator=g), torch.randn(T, W, generator=g)
    ctx = SimpleNamespace(step_tables={}, act_dtype=dt, stream_input=x0.cuda())
    for xx in (x, x * 2):                                    # twice a step: the x0 half is kept
        got = part.forward(ctx, xx.cuda().clone())
        assert got.dtype == torch.float32
        want = torch.cat([xx.to(dt).double(), x0.to(dt).double()], -1) @ w.double().T
        assert (got.double().cpu() - want).abs().max() < (2e-5 if dtype == "float32" else 1e-4) * float(want.abs().max() + 1)


# ====================================================================== the engine
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MZ_ALONE) + list(MZ_CONFIGS))
def test_whole_prompts_and_every_layer_run(mz_folders, name, dtype):
    """Logits at every position of whole prompts (the first tokens of a sequence among them),
    and the residual stream after every layer run, the loop's passes included."""
    cfg, weights = read_folder(mz_folders[name])
    reqs = _requests(cfg, [1, 2, 3, 41, 90], 100)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.whole(tb, rid, toks)
    core = _core(mz_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} whole")
    from helios_b200.engine.batch import StepEntry
    w = _bf16(weights) if dtype == "bfloat16" else weights
    _, _, want_layers = pm.forward(cfg, w, reqs["q3"], want_layers=True)
    seen = []

    def recording(inner):
        def forward(*args):
            residual, pending = inner(*args)
            x = residual.detach().double().cpu().clone()
            for t, s in pending.terms:
                x += pending.mult * t.double().cpu() * (1.0 if s is None else s.double().cpu())
            seen.append(x)
            return residual, pending
        return forward

    for blk in core.model.plan.layers:
        blk.forward = recording(blk.forward)
    core.step([StepEntry("layers", reqs["q3"], [0])])
    assert len(seen) == len(pm.layer_runs(cfg)) == want_layers.shape[0]
    for i, (got, want) in enumerate(zip(seen, want_layers)):
        tol = 2e-5 if dtype == "float32" else 3e-2 * float(want.abs().max())
        assert (got - want).abs().max() < tol, f"{name}: residual after layer run {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MZ_CONFIGS))
def test_prefill_then_long_decoding_token_by_token(mz_folders, name, dtype):
    """Most of the prompt in one step, then 70 single tokens (captured decode steps) that pass
    page borders and steps of the query temperature; every pass of the loop reads its own cache."""
    cfg, weights = read_folder(mz_folders[name])
    reqs = _requests(cfg, [75, 131, 260], 200)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.prefill_then_decode(tb, rid, toks, n_decode=70)
    core = _core(mz_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} decode")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MZ_CONFIGS))
def test_portions_of_changing_size_down_to_one_token(mz_folders, name, dtype):
    cfg, weights = read_folder(mz_folders[name])
    reqs = _requests(cfg, [64, 97, 50, 33], 300)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    sizes = [[7], [2, 31, 3, 16, 2, 17], [1, 2, 1, 1, 3, 13, 2, 1, 5], [16, 1, 15, 1]]
    for (rid, toks), sz in zip(reqs.items(), sizes):
        tu.portions(tb, rid, toks, sz)
    core = _core(mz_folders[name], dtype, tb.live_tokens_peak)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} portions")


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MZ_CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(mz_folders, name, dtype, graphs):
    """Nine unequal requests through three slots: portions of some beside single tokens of
    others; every finished request's pages and slot go to the next one."""
    cfg, weights = read_folder(mz_folders[name])
    reqs = _requests(cfg, [40, 23, 77, 18, 52, 31, 66, 20, 45], 400)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=7, max_live=3, decode_tail=10)
    core = _core(mz_folders[name], dtype, tb.live_tokens_peak, max_slots=3, graphs=graphs)
    tu.check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} mixed")
    assert core.cache.num_free_slots == 3 and all(p.num_used == 0 for p in core.cache.pools)


@pytest.mark.gpu
def test_a_batch_gives_each_request_what_it_gets_alone(mz_folders):
    """float32: the same rows bit for bit, alone or beside others, whatever the slots and pages."""
    from helios_b200.engine.batch import StepEntry

    cfg, _w = read_folder(mz_folders["mz_a"])
    reqs = _requests(cfg, [37, 5, 60], 500)
    core = _core(mz_folders["mz_a"], "float32", 512, max_slots=4)
    alone = {}
    for rid, toks in reqs.items():
        alone[rid] = core.step([StepEntry(rid, toks, range(len(toks)))]).clone()
        core.end(rid)
    core.step([StepEntry("other", random_tokens(cfg["vocab"], 21, 1), [0])])      # shifts slots and pages
    got = core.step([StepEntry(rid, toks, range(len(toks))) for rid, toks in reqs.items()])
    off = 0
    for rid, toks in reqs.items():
        assert torch.equal(got[off:off + len(toks)], alone[rid]), rid
        off += len(toks)


@pytest.mark.gpu
def test_a_request_may_not_pass_the_learned_positions(mz_folders):
    from helios_b200.engine.batch import StepEntry

    cfg, _w = read_folder(mz_folders["looped"])
    core = _core(mz_folders["looped"], "float32", 512)
    core.step([StepEntry("a", random_tokens(cfg["vocab"], 199, 1), [198])])
    core.step([StepEntry("a", [3], [0])])                  # position 199, the last one there is
    with pytest.raises(ValueError, match="max_model_len"):
        core.step([StepEntry("a", [3], [0])])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_through_trace_run(mz_folders, dtype, tmp_path):
    cfg, weights = read_folder(mz_folders["mz_b"])
    reqs = _requests(cfg, [30, 47, 22, 39, 28], 600)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=3, max_live=4, decode_tail=8)
    got = tu.run_trace_run(mz_folders["mz_b"], dtype, tb, tmp_path / "out", tb.live_tokens_peak, cfg["vocab"])
    tu.check(tb, got, plain, dtype, "mz_b trace_run")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(MZ_CONFIGS))
def test_greedy_generation_through_the_scheduler(mz_folders, name, dtype):
    from helios_b200 import LLM, SamplingParams

    cfg, weights = read_folder(mz_folders[name])
    w = _bf16(weights) if dtype == "bfloat16" else weights
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 5, 17, 33, 9, 26)]
    llm = LLM(str(mz_folders[name]), dtype=dtype, kv_cache_bytes=1 << 22, max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(max_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 12
        toks = list(prompt)
        for t in out.token_ids:
            logits = pm.forward(cfg, w, toks)[0][-1]
            best = int(torch.argmax(logits))
            if t != best:
                assert dtype == "bfloat16", f"token {t} instead of {best} after {len(toks)} tokens"
                assert float(logits[best] - logits[t]) <= 0.03 * float(logits.abs().max())
            toks.append(t)
