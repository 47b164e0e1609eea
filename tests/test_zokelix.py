"""The Zokelix design in the engine against the plain implementation (tests/plain_zokelix.py):
each mechanism alone, whole prompts, token-by-token decoding, portions down to one and two
tokens, mixed batches with pages and slots used again, ``bin/trace_run``, greedy generation
through the scheduler; plus kernel-level cases whose inputs make one far key, a page border
or the first token stand out.  Small configurations that differ in every size."""
from __future__ import annotations

import copy
import json
import math

import pytest
import torch

from conftest import random_tokens, read_folder
import plain_zokelix as pz
import trace_util as tu

DTYPES = ["float32", "bfloat16"]
YARN = {"factor": 4.0, "fast": 16.0, "slow": 2.0, "original": 64}


def _latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = scaling
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": scale, "rot": rot}}


def _delta(heads, kv_heads, dim, vdim, conv, low_rank):
    return {"type": "channel_delta",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                      "low_rank": low_rank}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def _model(vocab, width, eps, layers):
    return {"architecture": "Zokelix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(layer, mlp=mlp) for layer, mlp in layers]}


# Four layers, every kind of part, grouped q/k heads in the recurrent mixer, sizes that are
# no multiple of 32, two experts a token, a layer without a feed-forward.
ZK_A = _model(211, 96, 1e-5, [
    (_latent(3, 16, 8, 24, 40, 0.2, 10000.0, YARN), _dense(136)),
    (_delta(4, 2, 24, 40, 3, 16), _moe(48, 5, 2, 2.5)),
    (_delta(2, 2, 32, 16, 2, 8), None),
    (_latent(5, 24, 16, 8, 24, 0.11, 500000.0), _moe(48, 5, 2, 2.5)),
])
# Recurrent layer first, five taps, one and three experts a token, heads of 1, a latent wider
# than a head, a dense feed-forward behind a recurrent mixer, another eps.
ZK_B = _model(150, 80, 3e-6, [
    (_delta(1, 1, 40, 72, 5, 24), _dense(88)),
    (_latent(1, 8, 24, 40, 72, 0.3, 1000.0, {"factor": 16.0, "fast": 8.0, "slow": 1.0, "original": 32}), _moe(24, 3, 1, 0.7)),
    (_latent(4, 32, 8, 16, 16, 0.05, 10000.0), None),
    (_delta(6, 3, 16, 8, 4, 8), _moe(16, 7, 3, 1.0)),
])
ZK_CONFIGS = {"zk_a": ZK_A, "zk_b": ZK_B}
ZK_SEEDS = {"zk_a": 5, "zk_b": 6}
# one layer each: a mechanism alone
ZK_ALONE = {
    "latent_only": _model(97, 64, 1e-5, [(_latent(2, 16, 16, 24, 32, 0.17, 10000.0, YARN), None)]),
    "delta_only": _model(97, 64, 1e-5, [(_delta(2, 1, 16, 24, 4, 8), None)]),
    "dense_ff": _model(97, 64, 1e-5, [(_latent(2, 8, 8, 8, 16, 0.25), _dense(72))]),
    "routed_ff": _model(97, 64, 1e-5, [(_delta(2, 2, 8, 8, 2, 8), _moe(24, 6, 2, 1.5))]),
}


def _matrix_names(weights):
    return [k for k, v in weights.items() if v.dim() >= 2 and not k.endswith(".conv")]


def _bf16(weights):
    """What the bfloat16 path keeps: matrices rounded; vectors and convolution taps as stored."""
    names = set(_matrix_names(weights))
    return {k: (v.to(torch.bfloat16).float() if k in names else v) for k, v in weights.items()}


def _wide_router_margins(cfg, weights):
    """Make every routed layer's choice a matter of the token id with margins far beyond
    rounding, so that bfloat16 and float64 choose alike: channels 0..E-1 of the embedding
    hold a code (the token's j-th expert gets 4 - j), the norms leave those channels alone
    (weight 0 there, so the residual keeps the code exactly), and router row e reads the channels
    c with c % experts == e."""
    w = {k: v.clone() for k, v in weights.items()}
    E = max((l["mlp"]["router"]["experts"] for l in cfg["layers"] if l.get("mlp") and l["mlp"]["kind"] == "moe"),
            default=0)
    if not E:
        return w
    vocab = cfg["vocab"]
    w["embed"][:, :E] = 0.0
    for i, layer in enumerate(cfg["layers"]):
        for n in ("norm1", "norm2"):
            if f"l{i}.{n}" in w:
                w[f"l{i}.{n}"][:E] = 0.0
        ml = layer.get("mlp")
        if ml and ml["kind"] == "moe":
            e_here, top = ml["router"]["experts"], ml["router"]["top"]
            r = w[f"l{i}.mlp.router"]
            r[:, :E] = 0.0
            for c in range(E):
                r[c % e_here, c] = 2.0
    top_most = max(l["mlp"]["router"]["top"] for l in cfg["layers"] if l.get("mlp") and l["mlp"]["kind"] == "moe")
    for tok in range(vocab):
        for j in range(top_most):
            w["embed"][tok, (tok + j) % E] = 4.0 - j
    return w


@pytest.fixture(scope="module")
def zk_folders(tmp_path_factory):
    """name -> folder; the router margins are made wide, and ``low_rank`` is taken out of
    config.json again, so that the loader has to read it off the tensor shapes."""
    from safetensors.torch import save_file
    from helios_b200.weights import write_model_folder

    out = {}
    base = tmp_path_factory.mktemp("zokelix")
    for name, cfg in {**ZK_CONFIGS, **ZK_ALONE}.items():
        folder = write_model_folder(base / name, cfg, ZK_SEEDS.get(name, 9))
        _cfg, weights = read_folder(folder)
        save_file(_wide_router_margins(cfg, weights), str(folder / "model.safetensors"))
        stripped = copy.deepcopy(cfg)
        for layer in stripped["layers"]:
            layer["mixer"].pop("low_rank", None)
        with open(folder / "config.json", "w") as f:
            json.dump(stripped, f)
        out[name] = folder
    return out


def _plain(cfg, weights, dtype, requests):
    w = _bf16(weights) if dtype == "bfloat16" else weights
    return {rid: pz.forward_logits(cfg, w, toks) for rid, toks in requests.items()}


def _core(folder, dtype, max_tokens, page_size=16, max_slots=4, graphs=True):
    from helios_b200.engine.core import EngineCore
    from helios_b200.engine.model import DecoderModel

    model = DecoderModel.from_folder(folder, dtype=dtype)
    return EngineCore(model, page_size=page_size, num_pages=-(-max_tokens // page_size),
                      max_slots=max_slots, poison_cache=float("nan"), use_cuda_graphs=graphs)


# bfloat16 against the plain model on the rounded weights, row by row: the root mean square
# of the error (its mean taken off) over that of the logits.  Every sublayer's output is
# normalised before it is added, so its relative rounding error enters the residual stream
# undamped: under one per cent for the median row after four layers, but 6 % for a row where
# a sublayer's output nearly cancels before it is normalised, while a fault (a lost state, a
# stale page, a wrong slot) gives tens of per cent.  float32 keeps the 2e-5 of the other
# models' tests and is the sharp comparison.
ZK_BF16_RMS = 1e-1


def _check(tb, got, plain, dtype, what):
    if dtype == "float32":
        return tu.check(tb, got, plain, dtype, what)
    assert set(got) == set(tb.rows)
    for step, rows in tb.rows.items():
        want = torch.stack([plain[rid][pos] for rid, pos in rows])
        g = torch.from_numpy(got[step]).double()
        assert torch.isfinite(g).all(), f"{what} step {step}: non-finite logits"
        d = g - want
        d = d - d.mean(-1, keepdim=True)
        w = want - want.mean(-1, keepdim=True)
        rel = (d.pow(2).mean(-1) / w.pow(2).mean(-1)).sqrt()
        worst = int(rel.argmax())
        assert rel.max() <= ZK_BF16_RMS, (f"{what} step {step}: relative error {float(rel.max()):.3e} at "
                                          f"(request, position) {rows[worst]}; the step was {tb.steps[step]}")


def _requests(cfg, lengths, seed):
    return {f"q{i}": random_tokens(cfg["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ====================================================================== without a GPU
def test_configuration_is_read_layer_by_layer_and_faults_name_the_key():
    from helios_b200.config import ConfigError
    from helios_b200.config.registry import resolve_architecture
    from helios_b200.config.zokelix_config import ChannelDeltaConfig, LatentAttentionConfig, MoeMlpConfig

    arch = resolve_architecture(ZK_A)
    assert arch.name == "Zokelix"
    cfg = arch.parse_config(ZK_A)
    assert cfg.vocab_size == 211 and cfg.width == 96 and len(cfg.layers) == 4
    assert isinstance(cfg.layers[0].mixer, LatentAttentionConfig) and cfg.layers[0].mixer.rot.scaling.factor == 4.0
    assert isinstance(cfg.layers[1].mixer, ChannelDeltaConfig) and cfg.layers[1].mixer.kv_heads == 2
    assert isinstance(cfg.layers[1].mlp, MoeMlpConfig) and cfg.layers[1].mlp.top == 2 and cfg.layers[2].mlp is None
    assert cfg.layers[3].mixer.rot.scaling is None
    for path, value, word in ((("layers", 0, "type"), "conv_mixer", "type"),
                              (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mlp", "router", "top"), 9, "top"),
                              (("layers", 0, "mixer", "rot", "dims"), 7, "dims"),
                              (("norm",), {}, "eps")):
        bad = copy.deepcopy(ZK_A)
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=word):
            arch.parse_config(bad)


def test_plan_names_every_tensor_and_sizes_its_cache_and_state():
    from helios_b200.cache.manager import cache_groups_of
    from helios_b200.config.registry import resolve_architecture
    from helios_b200.weights.loader import expected_tensors

    arch = resolve_architecture(ZK_A)
    plan = arch.build_plan(arch.parse_config(ZK_A))
    names = expected_tensors(plan)
    assert names["embed"][2].shape == (211, 96) and names["head"][2].shape == (211, 96)
    assert names["final.norm"][2].shape == (96,) and names["l0.norm1"][2].shape == (96,)
    assert names["l0.mix.q"][2].shape == (3 * 24, 96) and names["l0.mix.dkv"][2].shape == (48, 96)
    assert names["l0.mix.uk"][2].shape == (48, 40) and names["l0.mix.uv"][2].shape == (72, 40)
    assert names["l0.mlp.gate.b"][2].shape == (136,) and names["l0.mlp.down.b"][2].shape == (96,)
    assert names["l1.mix.q"][2].shape == (48, 96) and names["l1.mix.v"][2].shape == (160, 96)
    assert names["l1.mix.k.conv"][2].shape == (48, 3) and names["l1.mix.a2"][2].shape == (96, 16)
    assert names["l1.mix.dt_bias"][2].shape == (96,) and names["l1.mix.A_log"][2].shape == (4,)
    assert names["l1.mlp.e4.down"][2].shape == (96, 48) and names["l1.mlp.router"][2].shape == (5, 96)
    assert "l2.norm2" not in names and "l2.mlp.router" not in names
    specs, where = cache_groups_of(plan)
    # one row a token: the latent and the shared rotated key part; two sizes, two groups
    assert [(s.num_kv_heads, s.head_dim, s.planes) for s in specs] == [(1, 48, 1), (1, 40, 1)]
    assert sorted(where) == [0, 3]
    d = plan.layers[1].mixer
    assert d.state_spec().shape == (4 * 24 * 40 + (2 * 48 + 160) * 2,)


def test_sizes_the_file_leaves_out_come_from_the_tensor_shapes(tmp_path):
    from helios_b200.config.registry import load_config
    from helios_b200.weights import write_model_folder

    folder = write_model_folder(tmp_path / "m", ZK_B, 3)
    stripped = copy.deepcopy(ZK_B)
    for layer in stripped["layers"]:
        layer["mixer"].pop("low_rank", None)
    with open(folder / "config.json", "w") as f:
        json.dump(stripped, f)
    cfg = load_config(folder)
    assert (cfg.layers[0].mixer.decay_rank, cfg.layers[0].mixer.gate_rank) == (24, 24)
    assert cfg.layers[3].mixer.decay_rank == 8


def test_yarn_frequencies_and_factor():
    from helios_b200.parts.rotary import yarn_attention_factor, yarn_frequencies

    for rot in ({"base": 10000.0, "dims": 8, "scaling": YARN},
                {"base": 250000.0, "dims": 48, "scaling": {"factor": 6.0, "fast": 24.0, "slow": 2.0, "original": 1024}},
                {"base": 1000.0, "dims": 24, "scaling": {"factor": 16.0, "fast": 8.0, "slow": 1.0, "original": 32}}):
        s = rot["scaling"]
        want, factor = pz.rotary_frequencies(rot)
        got = yarn_frequencies(rot["dims"], rot["base"], s["factor"], s["original"], s["fast"], s["slow"])
        assert torch.allclose(got, want, rtol=1e-14, atol=0)
        assert yarn_attention_factor(s["factor"]) == pytest.approx(factor, rel=1e-15)
        plain = rot["base"] ** (-2.0 * torch.arange(rot["dims"] // 2, dtype=torch.float64) / rot["dims"])
        assert torch.all(got <= plain * (1 + 1e-12)) and torch.all(got >= plain / s["factor"] * (1 - 1e-12))
    # some pair keeps its frequency and some pair is fully stretched in the first case
    got = yarn_frequencies(64, 10000.0, 4.0, 512, 32.0, 1.0)
    plain = 10000.0 ** (-2.0 * torch.arange(32, dtype=torch.float64) / 64)
    assert got[0] == plain[0] and got[-1] == pytest.approx(float(plain[-1]) / 4.0)


def test_toy_model_of_the_design_from_the_command_line(tmp_path):
    from helios_b200.cli import main

    out = tmp_path / "toy"
    assert main(["make-toy-model", "--arch", "zokelix", "--out", str(out), "--layers", "3", "--hidden-size", "48",
                 "--heads", "2", "--kv-heads", "1", "--vocab-size", "120"]) == 0
    cfg, weights = read_folder(out)
    assert cfg["architecture"] == "Zokelix" and [l["type"] for l in cfg["layers"]] == \
        ["latent_attention", "channel_delta", "latent_attention"]
    assert "l1.mix.A_log" in weights and "l2.mlp.router" in weights
    assert main(["info", "--model", str(out)]) == 0
    logits = pz.forward_logits(cfg, weights, [1, 2, 3])
    assert logits.shape == (3, 120) and torch.isfinite(logits).all()


# ====================================================================== kernels, inputs made to show faults
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_attention_kernel_far_key_page_borders_and_first_tokens(dtype):
    """One request of 300 tokens in pages of 16 handed out in a scrambled order.  A query's
    latent part is aligned with the row of ONE chosen key and scaled so that this key takes
    nearly all the weight: a far key among hundreds, the last key of a page, the first of the
    next, position 0, and the query's own position.  The kernel must return that key's latent."""
    from types import SimpleNamespace
    from helios_b200.csrc import ops

    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = "cuda"
    g = torch.Generator().manual_seed(3)
    n, page, rank, rot, heads = 300, 16, (40 if dtype == "float32" else 64), (8 if dtype == "float32" else 16), 3
    rows = torch.randn(n, rank + rot, generator=g)
    rows = (rows / rows.norm(dim=-1, keepdim=True)).to(dt).float()
    n_pages = -(-n // page)
    order = torch.randperm(n_pages + 3, generator=g)[:n_pages]
    pages = torch.full((n_pages + 4, 1, page, rank + rot), float("nan"), dtype=dt)
    for j in range(n):
        pages[order[j // page], 0, j % page] = rows[j].to(dt)
    cases = [(299, 2), (299, 15), (299, 16), (299, 0), (299, 299), (299, 287), (160, 159), (17, 16),
             (16, 16), (15, 0), (0, 0), (1, 0), (1, 1), (255, 31), (256, 32)]
    q_pos = torch.tensor([c[0] for c in cases], dtype=torch.int32)
    q = torch.zeros(len(cases), heads, rank + rot)
    for i, (_p, key) in enumerate(cases):
        for h in range(heads):
            q[i, h] = rows[key] * (40.0 + 10 * h)         # score 40..60 at the chosen key, |.| < that elsewhere
    q = q.to(dt)
    from helios_b200.engine.batch import SeqSlice
    # every query is a request of its own with one token, all reading the same pages
    ctx = SimpleNamespace(seq_of_token=torch.arange(len(cases), dtype=torch.int32, device=dev),
                          positions=q_pos.to(dev), start_pos=q_pos.to(dev), extras={}, max_context_len=n,
                          cu_tokens=torch.arange(len(cases) + 1, dtype=torch.int32, device=dev),
                          seqs=[SeqSlice(None, 0, p, 1, i) for i, (p, _k) in enumerate(cases)], num_seqs=len(cases))
    table = order.to(torch.int32).view(1, -1).repeat(len(cases), 1).contiguous().to(dev)
    qd = q.to(dev)
    out = ops.latent_attention(ctx, qd[:, :, :rank], qd[:, :, rank:], pages.to(dev), table, rank, rot, page, 1.0)
    out = out.float().cpu()
    for i, (pos, key) in enumerate(cases):
        s = torch.einsum("hd,jd->hj", q[i].double(), rows[:pos + 1].double())
        want = torch.softmax(s, -1) @ rows[:pos + 1, :rank].double()
        tol = 2e-5 if dtype == "float32" else 2e-2
        assert torch.isfinite(out[i]).all(), f"case {cases[i]}: read beyond position {pos}"
        assert (out[i].double() - want).abs().max() < tol, f"query at {pos}, key {key}"
        if pos != key or pos == 0:
            assert (out[i, -1].double() - rows[key, :rank].double()).abs().max() < 0.05


@pytest.mark.gpu
@pytest.mark.parametrize("heads,rank,rot", [(5, 160, 48), (40, 64, 16), (16, 256, 64), (3, 32, 0)])
def test_latent_attention_tensor_core_kernel_against_plain_softmax(heads, rank, rot):
    """bfloat16 sizes the tensor-core kernel takes: a decode batch of requests of unequal
    lengths (1, 2, 31, 32, 33, 300, 1000 keys; the key range cut into several blocks) and a
    portion of 77 tokens behind 200 cached ones, pages scattered, unwritten rows poisoned."""
    from types import SimpleNamespace
    from helios_b200.csrc import ops
    from helios_b200.engine.batch import SeqSlice

    dev, page = "cuda", 16
    g = torch.Generator().manual_seed(heads)
    lens = [1, 2, 31, 32, 33, 300, 1000]
    n_pages = sum(-(-n // page) for n in lens) + 20
    pages = torch.full((n_pages + 2, 1, page, rank + rot), float("nan"), dtype=torch.bfloat16)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lens)
    rows_of, table = [], torch.full((len(lens) + 1, width), -1, dtype=torch.int32)
    for i, n in enumerate(lens + [277]):
        rows = (torch.randn(n, rank + rot, generator=g) * 0.5).to(torch.bfloat16)
        rows_of.append(rows)
        if i == len(lens):
            table = torch.cat([table[:len(lens)], torch.full((1, width), -1, dtype=torch.int32)])
        for j in range(-(-n // page)):
            pg = order.pop()
            table[i, j] = pg
            chunk = rows[j * page:(j + 1) * page]
            pages[pg, 0, :len(chunk)] = chunk
    pages, table_d = pages.to(dev), table.contiguous().to(dev)

    def run(seq_ids, starts, counts, max_ctx):
        T = sum(counts)
        q = (torch.randn(T, heads, rank + rot, generator=g) * 0.7).to(torch.bfloat16)
        seq_of_token = torch.tensor([i for i, c in enumerate(counts) for _ in range(c)], dtype=torch.int32)
        positions = torch.tensor([s + k for s, c in zip(starts, counts) for k in range(c)], dtype=torch.int32)
        cu = torch.tensor([sum(counts[:i]) for i in range(len(counts) + 1)], dtype=torch.int32)
        ctx = SimpleNamespace(seq_of_token=seq_of_token.to(dev), positions=positions.to(dev), cu_tokens=cu.to(dev),
                              start_pos=torch.tensor(starts, dtype=torch.int32, device=dev), extras={},
                              seqs=[SeqSlice(None, 0, s, c, int(cu[i])) for i, (s, c) in enumerate(zip(starts, counts))],
                              max_context_len=max_ctx, num_seqs=len(counts))
        qd = q.to(dev)
        tab = table_d[seq_ids].contiguous()
        got = ops.latent_attention(ctx, qd[:, :, :rank], qd[:, :, rank:], pages, tab, rank, rot, page, 0.3)
        ops.LATENT_ATTENTION_TENSOR_CORES = False
        try:
            plain_kernel = ops.latent_attention(ctx, qd[:, :, :rank], qd[:, :, rank:], pages, tab, rank, rot, page, 0.3)
        finally:
            ops.LATENT_ATTENTION_TENSOR_CORES = True
        got, plain_kernel = got.float().cpu().double(), plain_kernel.float().cpu().double()
        assert torch.isfinite(got).all()
        t = 0
        for i, (sid, s0, c) in enumerate(zip(seq_ids, starts, counts)):
            rows = rows_of[sid].double()
            for k in range(c):
                sc = torch.einsum("hd,jd->hj", q[t].double(), rows[:s0 + k + 1]) * 0.3
                want = torch.softmax(sc, -1) @ rows[:s0 + k + 1, :rank]
                assert (got[t] - want).abs().max() < 2e-2, f"request {sid}, position {s0 + k}"
                assert (plain_kernel[t] - want).abs().max() < 2e-2
                t += 1

    run(list(range(len(lens))), [n - 1 for n in lens], [1] * len(lens), 1000)      # decode, ranges split
    run([len(lens)], [200], [77], 277)                                             # a portion behind a cached prefix
    run([5, 2, 6], [290, 0, 990], [10, 31, 10], 1000)                              # mixed


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_rule_kernel_against_the_scan_in_portions(dtype):
    """The recurrence kernel on two requests in slots 2 and 0, fed in portions of 1, 2, 17 and
    45 tokens, against the plain scan of the whole sequences; strong writes (beta near 1) and
    slow decays so that a token written long ago still shows at the end."""
    from types import SimpleNamespace
    from helios_b200.csrc import ops

    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = "cuda"
    g = torch.Generator().manual_seed(8)
    heads, kv_heads, dk, dv, n = 4, 2, 24, 40, 65
    lens = {"a": n, "b": n - 20}
    qk, C = kv_heads * dk, 2 * kv_heads * dk + heads * dv
    data = {r: dict(qkv=torch.randn(m, C, generator=g).to(dt), beta=(torch.randn(m, heads, generator=g) + 3).to(dt),
                    a=(torch.randn(m, heads * dk, generator=g) - 4).to(dt)) for r, m in lens.items()}
    a_log = torch.randn(heads, generator=g) * 0.3
    dt_bias = torch.randn(heads * dk, generator=g) * 0.3
    state = torch.full((4, heads * dk * dv + 5), float("nan"), device=dev)
    state[0].zero_()
    state[2].zero_()
    slots = {"a": 2, "b": 0}
    got = {r: [] for r in lens}
    fed = {r: 0 for r in lens}
    for sizes in ([1, 2], [2, 1], [17, 17], [45, 1], [0, 1], [0, 1], [0, 1], [0, 1]):
        parts = [(r, s) for r, s in zip(lens, sizes) if s and fed[r] < lens[r]]
        parts = [(r, min(s, lens[r] - fed[r])) for r, s in parts]
        cat = lambda k: torch.cat([data[r][k][fed[r]:fed[r] + s] for r, s in parts]).contiguous().to(dev)
        cu = torch.tensor([sum(s for _r, s in parts[:i]) for i in range(len(parts) + 1)], dtype=torch.int32, device=dev)
        ctx = SimpleNamespace(cu_tokens=cu, slots=torch.tensor([slots[r] for r, _s in parts], dtype=torch.int32, device=dev),
                              num_seqs=len(parts))
        o = ops.delta_rule(ctx, cat("qkv"), (0, qk, 2 * qk), cat("beta"), cat("a"), a_log.to(dev), dt_bias.to(dev),
                           state[:, :heads * dk * dv], heads, kv_heads, dk, dv).cpu()
        off = 0
        for r, s in parts:
            got[r].append(o[off:off + s])
            off += s
            fed[r] += s
    for r, m in lens.items():
        d = {k: v.double() for k, v in data[r].items()}
        q = d["qkv"][:, :qk].view(m, kv_heads, dk)
        k = d["qkv"][:, qk:2 * qk].view(m, kv_heads, dk)
        v = d["qkv"][:, 2 * qk:].view(m, heads, dv)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        beta = torch.sigmoid(d["beta"])
        gdec = torch.exp(-torch.exp(a_log.double())[None, :, None]
                         * torch.nn.functional.softplus(d["a"] + dt_bias.double()).view(m, heads, dk))
        have = torch.cat(got[r])[:fed[r]].double().view(-1, heads, dv)
        for h in range(heads):
            want = pz.delta_scan(q[:, h // 2], k[:, h // 2], v[:, h], beta[:, h], gdec[:, h])[:fed[r]]
            assert (have[:, h] - want).abs().max() < 2e-5, f"request {r}, head {h}"
    # nothing beyond the two slots' matrices was touched
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all() and float(state[[0, 2], -5:].abs().max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_short_convolution_carries_its_inputs_across_portions_shorter_than_its_taps(dtype):
    from types import SimpleNamespace
    from helios_b200.csrc import ops

    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = "cuda"
    g = torch.Generator().manual_seed(2)
    C, taps, n = 37, 5, 40
    x = torch.randn(n, C + 3, generator=g).to(dt)
    w = torch.randn(C, taps, generator=g)
    want = pz.short_conv_silu(x[:, :C].double(), w.double())
    state = torch.zeros(3, 7 + C * (taps - 1), device=dev)
    got, pos = [], 0
    for size in (1, 1, 2, 1, 3, 9, 2, 1, 1, 1, 4, 14):
        xs = x[pos:pos + size].contiguous().to(dev)
        ctx = SimpleNamespace(seq_of_token=torch.zeros(size, dtype=torch.int32, device=dev),
                              cu_tokens=torch.tensor([0, size], dtype=torch.int32, device=dev),
                              slots=torch.tensor([1], dtype=torch.int32, device=dev), num_seqs=1)
        got.append(ops.causal_conv_silu(ctx, xs, C, w.to(dev), state[:, 7:]).float().cpu())
        pos += size
    assert pos == n
    err = (torch.cat(got).double() - want).abs()
    assert (err.max() < 1e-5) if dtype == "float32" else bool((err <= 1e-2 * want.abs() + 1e-3).all())
    assert float(state[0].abs().max()) == 0 and float(state[2].abs().max()) == 0 and float(state[1, :7].abs().max()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("ff", [40, 20])
@pytest.mark.parametrize("dtype", DTYPES)
def test_router_and_experts_against_the_plain_functions(dtype, ff):
    """Same input for both sides, three of seven experts a token, a limit that clips.  An inner
    size of 20 is one the grouped product of the bfloat16 path does not take: every pair then
    streams its expert's rows, as in float32."""
    from helios_b200.csrc import ops

    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    dev = "cuda"
    g = torch.Generator().manual_seed(4)
    T, width, E, top, limit = 19, 72, 7, 3, 0.6
    h = torch.randn(T, width, generator=g).to(dt)
    W = {"router": (torch.randn(E, width, generator=g) * 0.2).to(dt).float()}
    for e in range(E):
        W[f"e{e}.gate"] = (torch.randn(ff, width, generator=g) * 0.2).to(dt).float()
        W[f"e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.2).to(dt).float()
        W[f"e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.2).to(dt).float()
    Wd = {k: v.double() for k, v in W.items()}
    ml = {"router": {"experts": E, "top": top}, "expert": {"ff": ff, "limit": limit}}
    want_ids, want_w = pz.router_choice(h.double(), Wd, "", top)
    logits = ops.linear_logits(h.to(dev), W["router"].to(dt).to(dev))
    ids, weights = ops.moe_topk(logits, top)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert (weights.cpu().double() - want_w).abs().max() < 1e-5
    w_gu = torch.stack([torch.cat([W[f"e{e}.gate"], W[f"e{e}.up"]]) for e in range(E)]).to(dt).to(dev)
    w_d = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(dt).to(dev)
    got = ops.moe_experts(h.to(dev), ids, weights, w_gu, w_d, limit).float().cpu().double()
    want = pz.routed_ff(h.double(), Wd, "", ml)
    tol = 2e-5 if dtype == "float32" else 3e-2 * float(want.abs().max())
    assert (got - want).abs().max() < tol


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_activations_and_the_norm_on_a_sublayer_output(dtype):
    from helios_b200.csrc import ops

    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    g = torch.Generator().manual_seed(6)
    gu = (torch.randn(11, 2 * 52, generator=g) * 2).to(dt)
    gate, up = gu[:, :52].double(), gu[:, 52:].double()
    tol = 1e-5 if dtype == "float32" else 3e-2
    got = ops.glu_act(gu.cuda(), "gelu_tanh").float().cpu().double()
    assert (got - pz.gelu_tanh(gate) * up).abs().max() < tol
    got = ops.glu_act(gu.cuda(), "clamped_swish", 1.25).float().cpu().double()
    gc, uc = gate.clamp(max=1.25), up.clamp(-1.25, 1.25)
    assert (got - gc * torch.sigmoid(1.702 * gc) * (uc + 1)).abs().max() < tol
    res = torch.randn(11, 52, generator=g)
    y = torch.randn(11, 52, generator=g).to(dt)
    w = torch.randn(52, generator=g)
    want = res.double() + pz.rms_norm(y.double(), w.double(), 1e-3)
    r = res.cuda()
    copy_ = ops.rmsnorm_add(r, y.cuda(), w.cuda(), 1e-3, dt)
    assert (r.cpu().double() - want).abs().max() < 1e-5          # the residual is float32 in both modes
    assert (copy_.float().cpu().double() - want).abs().max() < (1e-5 if dtype == "float32" else 3e-2)


# ====================================================================== the engine
@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ZK_ALONE) + list(ZK_CONFIGS))
def test_whole_prompts_and_every_layer(zk_folders, name, dtype):
    """Logits at every position of whole prompts (the first tokens of a sequence among them),
    and the residual stream after every layer."""
    cfg, weights = read_folder(zk_folders[name])
    reqs = _requests(cfg, [1, 2, 3, 41, 90], 100)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.whole(tb, rid, toks)
    core = _core(zk_folders[name], dtype, tb.live_tokens_peak)
    _check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} whole")
    # layer by layer
    from helios_b200.engine.batch import StepEntry
    w = _bf16(weights) if dtype == "bfloat16" else weights
    want_layers, _ = pz.forward_layers(cfg, w, reqs["q3"])
    seen = []

    def recording(inner):
        def forward(*args):
            residual, delta = inner(*args)
            seen.append(residual.detach().double().cpu().clone())
            return residual, delta
        return forward

    for blk in core.model.plan.layers:
        blk.forward = recording(blk.forward)
    core.step([StepEntry("layers", reqs["q3"], [0])])
    for i, (got, want) in enumerate(zip(seen, want_layers)):
        tol = 2e-5 if dtype == "float32" else 3e-2 * float(want.abs().max())
        assert (got - want).abs().max() < tol, f"{name}: residual after layer {i}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ZK_CONFIGS))
def test_prefill_then_long_decoding_token_by_token(zk_folders, name, dtype):
    """Most of the prompt in one step, then 70 single tokens (captured decode steps): the
    state of the recurrent layers and the latent cache carry on from token to token."""
    cfg, weights = read_folder(zk_folders[name])
    reqs = _requests(cfg, [75, 131], 200)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    for rid, toks in reqs.items():
        tu.prefill_then_decode(tb, rid, toks, n_decode=70)
    core = _core(zk_folders[name], dtype, tb.live_tokens_peak)
    _check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} decode")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ZK_CONFIGS))
def test_portions_of_changing_size_down_to_one_token(zk_folders, name, dtype):
    cfg, weights = read_folder(zk_folders[name])
    reqs = _requests(cfg, [64, 97, 50, 33], 300)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    sizes = [[7], [2, 31, 3, 16, 2, 17], [1, 2, 1, 1, 3, 13, 2, 1, 5], [16, 1, 15, 1]]
    for (rid, toks), sz in zip(reqs.items(), sizes):
        tu.portions(tb, rid, toks, sz)
    core = _core(zk_folders[name], dtype, tb.live_tokens_peak)
    _check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} portions")


@pytest.mark.gpu
@pytest.mark.parametrize("graphs", [True, False])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ZK_CONFIGS))
def test_mixed_batches_with_pages_and_slots_used_again(zk_folders, name, dtype, graphs):
    """Nine unequal requests through three slots: portions of some beside single tokens of
    others; every finished request's pages and slot go to the next one."""
    cfg, weights = read_folder(zk_folders[name])
    reqs = _requests(cfg, [40, 23, 77, 18, 52, 31, 66, 20, 45], 400)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=7, max_live=3, decode_tail=10)
    core = _core(zk_folders[name], dtype, tb.live_tokens_peak, max_slots=3, graphs=graphs)
    _check(tb, tu.run_in_process(core, tb), plain, dtype, f"{name} mixed")
    assert core.cache.num_free_slots == 3 and all(p.num_used == 0 for p in core.cache.pools)


@pytest.mark.gpu
def test_a_batch_gives_each_request_what_it_gets_alone(zk_folders):
    """float32: the same rows bit for bit, alone or beside others, whatever the slots and pages."""
    from helios_b200.engine.batch import StepEntry

    cfg, _w = read_folder(zk_folders["zk_a"])
    reqs = _requests(cfg, [37, 5, 60], 500)
    core = _core(zk_folders["zk_a"], "float32", 512, max_slots=4)
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
@pytest.mark.parametrize("dtype", DTYPES)
def test_through_trace_run(zk_folders, dtype, tmp_path):
    cfg, weights = read_folder(zk_folders["zk_b"])
    reqs = _requests(cfg, [30, 47, 22, 39, 28], 600)
    plain = _plain(cfg, weights, dtype, reqs)
    tb = tu.TraceBuilder()
    tu.mixed(tb, reqs, seed=3, max_live=4, decode_tail=8)
    got = tu.run_trace_run(zk_folders["zk_b"], dtype, tb, tmp_path / "out", tb.live_tokens_peak, cfg["vocab"])
    _check(tb, got, plain, dtype, "zk_b trace_run")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ZK_CONFIGS))
def test_greedy_generation_through_the_scheduler(zk_folders, name, dtype):
    from helios_b200 import LLM, SamplingParams

    cfg, weights = read_folder(zk_folders[name])
    w = _bf16(weights) if dtype == "bfloat16" else weights
    prompts = [random_tokens(cfg["vocab"], n, 40 + n) for n in (1, 5, 17, 33, 9, 26)]
    llm = LLM(str(zk_folders[name]), dtype=dtype, kv_cache_bytes=1 << 22, max_num_batched_tokens=24,
              max_num_seqs=4, max_model_len=256)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(max_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out.completion_tokens == 12
        toks = list(prompt)
        for t in out.token_ids:
            logits = pz.forward_logits(cfg, w, toks)[-1]
            best = int(torch.argmax(logits))
            if t != best:
                assert dtype == "bfloat16", f"token {t} instead of {best} after {len(toks)} tokens"
                assert float(logits[best] - logits[t]) <= 0.03 * float(logits.abs().max())
            toks.append(t)
