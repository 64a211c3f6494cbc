"""The Demavik decoder through the engine against the plain implementation (tests/plain_demavik.py).

Small configurations of their own sizes and random weights, made here.  On a GPU the engine runs its CUDA kernels in
float32 and bfloat16; without one the same tests run the host-side logic (configuration, loader, cache manager with
pages and state slots, step function) over the kernels' plain references.  Covered: each mechanism alone; a prompt
whole, against its last tokens decoded one by one, against portions down to two tokens and one; long portions whose
scans run in chunks; unequal requests in one batch against each alone, with pages and slots that are given back and
used again; the first tokens of a sequence (the pair embedding's own row, the previous token across steps); a token
far back that only the recurrent states and a far key carry; a far key with one score made to stand out, at page
borders, in prompts and in decoding; long decoding from captured steps; a configuration of ones; greedy generation
through the front end; configuration errors; random-weights mode; each new kernel against its plain reference.
"""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_demavik as P
from helpers import random_tokens

CUDA = torch.cuda.is_available()
DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]
DTYPES = ["float32", "bfloat16"]


def moe(experts=5, top=2, ff=24):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def attention(heads=6, kv=2, dim=16, vdim=32, rot=8, base=900.0, scaling=(8.0, 1.0, 4.0, 64), scale=0.31, kv_from=None, mlp=None):
    r = {"dims": rot, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "rot": r, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def gla(heads=3, dim=16, vdim=24, tau=4.0, mlp=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def mamba(inner=40, state=12, dt_rank=3, conv=4, mlp=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, mult=0.7, scale=2.5, bigram=(13, 31, 7)):
    emb = {"scale": scale}
    if bigram:
        emb["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return {"architecture": "Demavik", "embedding": emb, "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
            "width": width}


# ranks of the decays' maps: config.json does not give them, the stored shape does (layer index -> rank)
RANKS = {"mixed": {2: 5}, "gla_only": {0: 7}, "ones": {1: 1}, "far": {0: 4}, "shared_first": {1: 3}, "odd": {1: 3}, "wide": {0: 8}}

CONFIGS = {
    # everything at once, no two sizes alike: value heads wider and narrower than key heads, three query heads per key
    # head, part of a head rotated with scaled and unscaled frequencies, a layer that reads another's keys and values with
    # a layer of another kind in between, several experts per token, layers without feed-forward
    "mixed": config([
        attention(mlp=moe(5, 2, 24)),
        mamba(mlp=None),
        gla(mlp=moe(3, 1, 40)),
        attention(kv_from=0, mlp=moe(4, 4, 16)),
        attention(heads=2, kv=2, dim=32, vdim=16, rot=32, base=10000.0, scaling=None, scale=0.2, mlp=None),
    ]),
    # each mechanism alone
    "attention_only": config([attention(mlp=None)], width=32, vocab=61, bigram=None),
    "shared_only": config([attention(heads=4, kv=1, dim=16, vdim=16, rot=16, mlp=None), attention(heads=4, kv=1, dim=16, vdim=16, rot=16, kv_from=0, mlp=None)],
                          width=32, vocab=61, bigram=None, scale=1.0),
    "gla_only": config([gla(mlp=None)], width=32, vocab=61, bigram=None),
    "mamba_only": config([mamba(mlp=None)], width=32, vocab=61, bigram=None, mult=1.0),
    "experts_only": config([gla(heads=1, dim=8, vdim=8, tau=2.0, mlp=moe(6, 3, 20))], width=40, vocab=50, eps=1e-6, bigram=None),
    "pairs_only": config([mamba(inner=16, state=4, dt_rank=2, conv=2, mlp=None)], width=24, vocab=40, bigram=(7, 3, 5)),
    # another order: the state-space layer first, the sharing layers next to each other at the end
    "shared_first": config([mamba(inner=24, state=33, dt_rank=2, conv=3, mlp=moe(2, 1, 8)), gla(heads=2, dim=40, vdim=8, tau=9.0, mlp=None),
                            attention(heads=2, kv=1, dim=16, vdim=24, rot=4, mlp=None), attention(heads=2, kv=1, dim=16, vdim=24, rot=4, kv_from=2, mlp=moe(3, 2, 8))],
                           width=40, vocab=33, bigram=(1, 1, 1), mult=0.25, scale=0.5),
    # values that a model may happen to make equal or 1: one head, one expert, one tap, a state of one, a rank of one, no
    # factor on the stream or the embedding, one bucket
    "ones": config([attention(heads=1, kv=1, dim=16, vdim=16, rot=2, scaling=None, scale=1.0, mlp=moe(1, 1, 8)),
                    gla(heads=1, dim=8, vdim=8, tau=1.0, mlp=None), mamba(inner=8, state=1, dt_rank=1, conv=1, mlp=None)],
                   width=16, vocab=17, mult=1.0, scale=1.0, bigram=(1, 2, 3)),
    # sizes that are multiples of nothing much: a width of 36, heads of 12, 20, 10 and 6, 18 channels with a state of 5
    "odd": config([attention(heads=3, kv=1, dim=12, vdim=20, rot=6, scale=0.4, mlp=moe(3, 2, 12)), gla(heads=2, dim=10, vdim=6, tau=3.0, mlp=None),
                   mamba(inner=18, state=5, dt_rank=3, conv=2, mlp=moe(3, 2, 12)), attention(heads=3, kv=1, dim=12, vdim=20, rot=6, scale=0.4, kv_from=0, mlp=None)],
                  width=36, vocab=35, bigram=(11, 5, 3)),
    # sizes of a model's layers, where the tensor-core kernels take the heads (64 and 128) and the experts' products
    "wide": config([gla(heads=2, dim=64, vdim=128, tau=8.0, mlp=moe(8, 2, 64)),
                    attention(heads=4, kv=2, dim=64, vdim=64, rot=64, base=10000.0, scaling=(4.0, 1.0, 4.0, 256), scale=0.125, mlp=moe(8, 2, 64)),
                    attention(heads=4, kv=2, dim=64, vdim=64, rot=64, base=10000.0, scaling=(4.0, 1.0, 4.0, 256), scale=0.125, kv_from=1, mlp=None),
                    mamba(inner=512, state=16, dt_rank=16, conv=4, mlp=moe(8, 2, 64)),
                    attention(heads=2, kv=1, dim=128, vdim=128, rot=32, base=50000.0, scaling=None, scale=0.09, mlp=None)],
                   width=256, vocab=512, mult=0.5, scale=3.0, bigram=(509, 127, 17)),
    # states that forget slowly (see make_weights) and full attention: a token far back still moves the last logits
    "far": config([gla(heads=2, dim=16, vdim=16, tau=16.0, mlp=None), attention(heads=2, kv=1, dim=16, vdim=16, rot=16, mlp=None)],
                  width=32, vocab=41),
}


def with_ranks(name, cfg):
    """config.json with the decays' ranks written into it, for the plain side and the declared tensors."""
    cfg = json.loads(json.dumps(cfg))
    for i, r in RANKS.get(name, {}).items():
        cfg["layers"][i]["mixer"]["decay_rank"] = r
    return cfg


def declared(name):
    from litinfer_b200.config import config_from_dict
    from litinfer_b200.models.decoder import declared_params

    return declared_params(config_from_dict(with_ranks(name, CONFIGS[name])).to_model_spec())


def make_weights(name, seed):
    """Random tensors for every declared name, large enough that each part moves the logits."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for p in declared(name):
        n, shape = p.name, tuple(p.shape)
        r = torch.randn(shape, generator=g)
        last = n.rsplit(".", 1)[-1]
        if last in ("norm", "norm1", "norm2") or n.endswith("q.norm") or n.endswith("k.norm") or last == "D":
            out[n] = 1.0 + 0.2 * r
        elif n.endswith("a2.b"):
            out[n] = (6.0 if name == "far" else 1.5) + 0.5 * r          # "far": decays near one, the state forgets slowly
        elif n.endswith("dt.b"):
            out[n] = -1.0 + 0.5 * r
        elif last == "b":
            out[n] = 0.3 * r
        elif last == "conv":
            out[n] = 0.6 * r
        elif last == "A_log":
            out[n] = 0.5 * r - (2.0 if name == "far" else 0.0)
        elif last == "router":
            out[n] = r * (3.0 / math.sqrt(shape[-1]))
        elif n == "embed":
            out[n] = r
        elif n == "bigram":
            out[n] = 0.7 * r
        else:
            out[n] = r * (1.5 / math.sqrt(shape[-1]))
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from litinfer_b200.weights.safetensors_io import write_file

    out = {}
    for k, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp("demavik_" + name)
        w = make_weights(name, 191 + k)
        (d / "config.json").write_text(json.dumps(cfg))           # without the ranks: the engine reads them off the shapes
        write_file(d / "model.safetensors", w)
        out[name] = (d, with_ranks(name, cfg), w)
    return out


def use_device(device, request):
    if device == "cpu":
        request.getfixturevalue("cpu_kernels")
    return torch.device("cuda:0" if device == "cuda" else "cpu")


def oracle(name, cfg, w, tokens, dtype, keep=None):
    if dtype == "bfloat16":
        # what the bfloat16 engine holds: matrices rounded to bfloat16, everything else in float32
        roles = {p.name: p.role for p in declared(name)}
        w = {k: (v.to(torch.bfloat16).float() if roles[k] == "matrix" else v) for k, v in w.items()}
    return P.forward(cfg, {k: v.double() for k, v in w.items()}, tokens, keep).float()


def assert_close(got, ref, dtype, what):
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    err = d.pow(2).mean(dim=-1).sqrt() / ref.std(dim=-1).clamp_min(1e-3)
    worst = int(err.argmax())
    if dtype == "float32":
        assert err.max() <= 2e-4, f"{what}: relative error {float(err.max()):.3e} at row {worst}"
        return
    # bfloat16: activations are rounded to 8 bits at a dozen places a layer.  A row may be unlucky, and a token whose two
    # best experts score within that rounding of each other may go to the other one than in the plain model; most rows may
    # not (a wrong key, a lost state or a wrong previous token moves every row behind it by tens of percent)
    assert err.median() <= 0.05, f"{what}: median relative error {float(err.median()):.3e}"
    assert (err > 0.2).float().mean() <= 0.15, f"{what}: {int((err > 0.2).sum())} of {err.numel()} rows are off, the worst ({worst}) by {float(err.max()):.3e}"


class Run:
    """Feeds requests to a Replayer step by step and keeps every position's logits."""

    def __init__(self, folder, dtype, device, max_tokens, max_live=4, graphs=None):
        from litinfer_b200.engine.replay import Replayer
        from litinfer_b200.models import DecoderModel

        self.model = DecoderModel.from_dir(folder, dtype, device)
        self.rp = Replayer(self.model, max_tokens, max_live=max_live, use_graphs=device.type == "cuda" if graphs is None else graphs)
        self.fed = {}
        self.got = {}
        self.n = 0

    def step(self, entries, end=()):
        """entries: (request, all its tokens, how many of them now)."""
        es = []
        for rid, tokens, count in entries:
            lo = self.fed.get(rid, 0)
            es.append({"id": rid, "tokens": tokens[lo:lo + count], "want": list(range(count))})
            self.fed[rid] = lo + count
        logits = self.rp.step({"step": self.n, "entries": es, "end": list(end)}).float().cpu()
        self.n += 1
        row = 0
        for (rid, tokens, count), e in zip(entries, es):
            self.got.setdefault(rid, []).append(logits[row:row + count])
            row += count
        for rid in end:
            self.fed.pop(rid)

    def logits(self, rid):
        return torch.cat(self.got[rid])


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention_only", "shared_only", "gla_only", "mamba_only", "experts_only", "pairs_only", "ones", "shared_first"])
def test_each_mechanism_alone(name, dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders[name]
    toks = random_tokens(45, cfg["vocab"], 5)
    ref = oracle(name, cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 128)
    run.step([("a", toks, 45)], end=["a"])
    assert_close(run.logits("a"), ref, dtype, f"{name} whole")
    run.step([("b", toks, 30)])
    for _ in range(15):
        run.step([("b", toks, 1)])
    assert_close(run.logits("b"), ref, dtype, f"{name} decoded")
    # portions of two tokens from the start: the states, the convolution's inputs and the previous token cross every step
    for i in range(10):
        run.step([("c", toks, 2)])
    assert_close(run.logits("c"), ref[:20], dtype, f"{name} in twos")


@pytest.mark.parametrize("device", DEVICES)
def test_the_residual_stream_after_every_layer(device, folders, request):
    """Float32, layer by layer: the stream after each block against the plain model's."""
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    toks = random_tokens(37, cfg["vocab"], 8)
    keep = []
    oracle("mixed", cfg, w, toks, "float32", keep)
    run = Run(folder, "float32", dev, 64, graphs=False)
    seen = []
    run.model.observer = lambda i, x, carry: seen.append(x.detach().float().cpu().clone())
    run.step([("a", toks, 37)])
    assert len(seen) == len(keep) == 5
    for i, (a, b) in enumerate(zip(seen, keep)):
        assert (a - b.float()).abs().max() <= 1e-4 * max(1.0, float(b.abs().max())), f"after layer {i}"


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_whole_decoded_and_in_portions(dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    n = 300 if device == "cuda" else 150
    toks = random_tokens(n, cfg["vocab"], 11)
    ref = oracle("mixed", cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 320)
    run.step([("whole", toks, n)], end=["whole"])                  # (a portion of 128 tokens and more: the scans run in chunks of 64)
    assert_close(run.logits("whole"), ref, dtype, "whole")
    # most of it at once, then token by token across page borders (16) and chunk borders
    run.step([("tail", toks, n - 50)])
    for i in range(50):
        run.step([("tail", toks, 1)], end=["tail"] if i == 49 else [])
    assert_close(run.logits("tail"), ref, dtype, "decoded")
    # portions of changing size, down to two tokens and one, one of them long enough for chunks; the first token alone
    fed, i, sizes = 0, 0, [1, 2, 7, 16, 2, 33, 5, 2, 130, 3, 1, 2, 11, 2, 29]
    while fed < n:
        c = min(sizes[i % len(sizes)], n - fed)
        run.step([("cut", toks, c)], end=["cut"] if fed + c == n else [])
        fed += c
        i += 1
    assert_close(run.logits("cut"), ref, dtype, "portions")
    # token by token from the very first one
    for i in range(40):
        run.step([("one", toks, 1)], end=["one"] if i == 39 else [])
    assert_close(run.logits("one"), ref[:40], dtype, "token by token from the start")
    if dtype == "float32":
        assert (run.logits("whole") - run.logits("cut")).abs().max() < 1e-4
        assert (run.logits("whole") - run.logits("tail")).abs().max() < 1e-4
    run.rp.manager.check()
    assert run.rp.manager.num_free_slots() == 4


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_other_sizes_whole_decoded_and_in_portions(name, dtype, device, folders, request):
    """Sizes that are multiples of nothing, and sizes of a real model's layers (on a GPU: the kernels for heads of 64 and
    128, for long portions and for many experts' rows): a prompt whole, its end decoded, and in portions."""
    dev = use_device(device, request)
    folder, cfg, w = folders[name]
    n = 330 if device == "cuda" else 70
    toks = random_tokens(n, cfg["vocab"], 23)
    ref = oracle(name, cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 384)
    run.step([("whole", toks, n)], end=["whole"])
    assert_close(run.logits("whole"), ref, dtype, f"{name} whole")
    run.step([("tail", toks, n - 40)])
    for i in range(40):
        run.step([("tail", toks, 1)], end=["tail"] if i == 39 else [])
    assert_close(run.logits("tail"), ref, dtype, f"{name} decoded")
    fed, i, sizes = 0, 0, [3, 64, 2, 129, 17, 1, 70]
    while fed < n:
        c = min(sizes[i % len(sizes)], n - fed)
        run.step([("cut", toks, c)], end=["cut"] if fed + c == n else [])
        fed += c
        i += 1
    assert_close(run.logits("cut"), ref, dtype, f"{name} portions")
    if dtype == "float32":
        assert (run.logits("whole") - run.logits("cut")).abs().max() < 2e-4
    run.rp.manager.check()


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(dtype, device, folders, request):
    dev = use_device(device, request)
    folder, cfg, w = folders["mixed"]
    lens = [150, 37, 1, 64, 23, 2, 55, 140] if device == "cuda" else [40, 17, 1, 33, 2, 21]
    reqs = {f"r{j}": random_tokens(n, cfg["vocab"], 40 + j) for j, n in enumerate(lens)}
    # a pool for the most tokens that are live at a time, each request rounded up to 64: pages and slots come back
    run = Run(folder, dtype, dev, 64 * 7, max_live=3)
    queue, live, step_no = list(reqs), [], 0
    portions = [5, 2, 16, 9, 3, 21, 2, 130]
    while queue or live:
        while queue and len(live) < 3:
            live.append(queue.pop(0))
        entries, ending = [], []
        for k, rid in enumerate(live):
            toks, fed = reqs[rid], run.fed.get(rid, 0)
            if (step_no + k) % 5 == 4 and fed > 0:
                continue                                    # left out of this step, goes on later
            c = min(portions[(step_no + k) % len(portions)], len(toks) - fed) if fed < 0.6 * len(toks) else 1
            entries.append((rid, toks, c))
            if fed + c == len(toks):
                ending.append(rid)
        if entries:
            run.step(entries, end=ending)
        live = [r for r in live if r not in ending]
        step_no += 1
    if dtype == "float32":
        for rid, toks in reqs.items():
            assert_close(run.logits(rid), oracle("mixed", cfg, w, toks, dtype), dtype, f"{rid} of {len(toks)} tokens in mixed batches")
    else:
        alone = Run(folder, dtype, dev, 64 * 7, max_live=3)
        for rid, toks in reqs.items():
            alone.step([(rid, toks, len(toks))], end=[rid])
            assert_close(run.logits(rid), alone.logits(rid), dtype, f"{rid} of {len(toks)} tokens: in mixed batches against alone")
        assert_close(torch.cat([run.logits(r) for r in reqs]), torch.cat([oracle("mixed", cfg, w, t, dtype) for t in reqs.values()]), dtype, "all requests")
    m = run.rp.manager
    m.check()
    assert m.num_free_slots() == 3 and all(m.num_free_pages(g) == m.num_pages for g in range(len(m.groups)))


@pytest.mark.parametrize("device", DEVICES)
def test_a_token_far_back_reaches_the_last_logits_through_the_states_and_a_far_key(device, folders, request):
    """Two prompts that differ in their first token only.  With decays near one and full attention the last logits still
    differ, in the plain model and in the engine alike, whole (scans in chunks) and decoded one by one."""
    dev = use_device(device, request)
    folder, cfg, w = folders["far"]
    n = 260 if device == "cuda" else 140
    a = random_tokens(n, cfg["vocab"], 21)
    b = [(a[0] + 1) % cfg["vocab"]] + a[1:]
    ra, rb = oracle("far", cfg, w, a, "float32"), oracle("far", cfg, w, b, "float32")
    moved = float((ra[-1] - rb[-1]).abs().max())
    assert moved > 1e-2, "the plain model has forgotten the first token: make the decays slower"
    run = Run(folder, "float32", dev, 64 * 10)
    run.step([("a", a, n)], end=["a"])
    run.step([("b", b, n - 20)])
    for i in range(20):
        run.step([("b", b, 1)], end=["b"] if i == 19 else [])
    assert_close(run.logits("a"), ra, "float32", "first prompt")
    assert_close(run.logits("b"), rb, "float32", "second prompt")
    assert float((run.logits("a")[-1] - run.logits("b")[-1]).abs().max()) > 0.5 * moved


@pytest.mark.parametrize("device", DEVICES)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("q_len", [1, 7, 70])
def test_a_far_key_among_hundreds_with_one_score_made_to_stand_out(q_len, dtype, device, request):
    """Full causal attention (no window), kernel level: every query has a large component along one key, at the very
    start, at a page border, or right before it; that key's value is a marker that must reach the output."""
    dev = use_device(device, request)
    from litinfer_b200 import kernels as K

    nh, nkv, dh, page = 4, 2, 32, 16
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    for ctx in ([75, 700] if device == "cuda" else [75]):
        for hot in (0, 15, 16, ctx - q_len - 1, ctx - 1):
            torch.manual_seed(ctx + hot)
            k, v, q = 0.05 * torch.randn(ctx, nkv, dh), 0.05 * torch.randn(ctx, nkv, dh), 0.05 * torch.randn(q_len, nh, dh)
            k[hot, :, 3] += 6.0
            q[:, :, 3] += 6.0
            v[hot, :, 0] = 10.0
            pages = -(-ctx // page)
            order = torch.randperm(pages)
            kc, vc = torch.zeros(pages + 1, nkv, page, dh), torch.zeros(pages + 1, nkv, dh, page)
            for j in range(ctx):
                kc[order[j // page], :, j % page] = k[j]
                vc[order[j // page], :, :, j % page] = v[j]
            qkv = torch.cat([q.reshape(q_len, -1), torch.zeros(q_len, 2 * nkv * dh)], dim=1).to(dev, dt).contiguous()
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
            out = torch.empty(q_len, nh * dh, dtype=dt, device=dev)
            K.paged_attention(qkv, out, kc.to(dev, dt), vc.to(dev, dt), order.to(torch.int32).view(1, -1).to(dev).contiguous(), i32([0, q_len]),
                              i32([ctx]), i32([0] * q_len), i32(list(range(ctx - q_len, ctx))), nh, nkv, dh, 1.0, None, q_len, ctx)
            got = out.float().cpu().view(q_len, nh, dh)[:, :, 0]
            for t in range(q_len):
                seen = hot <= ctx - q_len + t
                assert (got[t].min() > 5.0) == seen, f"ctx {ctx}, {q_len} tokens, token {t}: key {hot} {'is' if seen else 'is not'} seen"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_captured_steps(dtype, folders):
    """300 tokens one by one (steps replayed from a captured graph: states, convolution inputs, previous tokens and pages
    moving on) against the prompt whole."""
    folder, cfg, w = folders["mixed"]
    toks = random_tokens(330, cfg["vocab"], 3)
    ref = oracle("mixed", cfg, w, toks, dtype)
    run = Run(folder, dtype, torch.device("cuda:0"), 384)
    run.step([("a", toks, 30)])
    for _ in range(300):
        run.step([("a", toks, 1)])
    assert run.rp.runner.graph_replays >= 290
    assert_close(run.logits("a"), ref, dtype, "long decoding")


@pytest.mark.parametrize("device", DEVICES)
def test_greedy_generation_through_the_front_end(device, folders, request):
    dev = use_device(device, request)
    from litinfer_b200.api import CausalLM
    from litinfer_b200.models import DecoderModel

    folder, cfg, w = folders["mixed"]
    w64 = {k: v.double() for k, v in w.items()}
    lm = CausalLM(folder, dtype="float32") if device == "cuda" else CausalLM(folder, device="cpu", model=DecoderModel.from_dir(folder, "float32", dev),
                                                                            use_graphs=False)
    for n, new in ((1, 6), (13, 20), (50, 12)):
        prompt = random_tokens(n, cfg["vocab"], 60 + n)
        toks, margins = list(prompt), []
        for _ in range(new):
            top = torch.topk(P.forward(cfg, w64, toks)[-1], 2)
            margins.append(float(top.values[0] - top.values[1]))
            toks.append(int(top.indices[0]))
        assert min(margins) > 1e-4, "the plain model's own choice is a near-tie; pick another seed"
        out = lm.generate(prompt, max_new_tokens=new)
        assert list(out)[-new:] == toks[n:], f"prompt of {n} tokens"


def test_configuration_is_read_and_refused():
    from litinfer_b200.config import ConfigError, config_from_dict
    from litinfer_b200.parts.rope import scaled_denominators

    cfg = with_ranks("mixed", CONFIGS["mixed"])
    spec = config_from_dict(cfg).to_model_spec()
    assert len(spec.blocks) == 5 and [e.cache_from for e in spec.schedule] == [None, None, None, 0, None]
    assert spec.embedding_scale == 2.5 and spec.stream_inputs[0][0]["buckets"] == 13
    att, shared = spec.blocks[0].parts["mixer"], spec.blocks[3].parts["mixer"]
    assert att["value_dim"] == 32 and att["position"]["rotary_dim"] == 8 and att["qk_norm"]["whole"] and not att["shared_kv"] and shared["shared_kv"]
    assert spec.blocks[2].parts["mixer"]["decay_rank"] == 5 and spec.blocks[1].parts["mixer"]["state_size"] == 12
    ff = spec.blocks[0].parts["feed_forward"]
    assert ff["experts"] == 5 and ff["top"] == 2 and ff["weight_on"] == "output" and ff["scoring"] == "softmax_chosen" and "feed_forward" not in spec.blocks[1].parts
    assert spec.blocks[0].parts["mixer_post_norm"]["gain"] == 0.7 and spec.blocks[0].parts["mixer_norm"].kind == "identity"
    # the scaled frequencies against the plain model's: kept, blended and divided ones are all there
    rot = cfg["layers"][0]["mixer"]["rot"]
    mine = torch.tensor(scaled_denominators(rot["base"], rot["dims"], rot["scaling"]), dtype=torch.float64)
    plain = 1.0 / P.rotary_frequencies(rot)
    unscaled = torch.tensor([rot["base"] ** (2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
    assert torch.allclose(mine, plain, rtol=1e-12)
    ratio = (mine / unscaled).tolist()
    assert ratio[0] == 1.0 and 1.0 < ratio[1] < 8.0 and abs(ratio[2] - 8.0) < 1e-9 and abs(ratio[3] - 8.0) < 1e-9
    for path, bad in ((("layers", 0, "type"), "mamba2"), (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mixer", "kv_heads"), 4),
                      (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mlp", "router", "top"), 9), (("layers", 3, "mixer", "kv_from"), 1),
                      (("layers", 3, "mixer", "kv_from"), 3), (("layers", 3, "mixer", "heads"), 2), (("layers", 0, "mixer", "rot", "scaling", "high"), 0.5),
                      (("layers", 1, "mixer", "state"), 0), (("embedding", "bigram", "buckets"), 0), (("norm",), None), (("width",), 0)):
        broken = json.loads(json.dumps(cfg))
        at = broken
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = bad
        with pytest.raises(ConfigError):
            config_from_dict(broken)


def test_random_weights_and_a_written_folder(tmp_path, cpu_kernels):
    """Random-weights mode knows the design's tensors: a folder written from the configuration loads and steps."""
    from litinfer_b200.weights import write_model_folder
    from litinfer_b200.weights.safetensors_io import iter_tensors, read_header

    cfg = with_ranks("mixed", CONFIGS["mixed"])
    d = write_model_folder(tmp_path / "m", dict(cfg), seed=5)
    header, _ = read_header(d / "model.safetensors")
    w = {n: t.double() for n, t in iter_tensors(d / "model.safetensors", set(header))}
    assert w["bigram"].shape == (14, 48) and w["l2.mix.a1"].shape == (5, 48) and w["l1.mix.A_log"].shape == (40, 12) and "l3.mix.k" not in w
    toks = random_tokens(20, cfg["vocab"], 1)
    run = Run(d, "float32", torch.device("cpu"), 64)
    run.step([("a", toks, 20)])
    assert_close(run.logits("a"), P.forward(cfg, w, toks).float(), "float32", "written folder")


# --------------------------------------------------------------------------
# each new kernel alone against its plain float32 reference (tests/kernel_refs.py)
# --------------------------------------------------------------------------

def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(a, b, dtype, what, tol=None):
    a, b = a.float().cpu(), b.float().cpu()
    tol = tol or (3e-5 if dtype == "float32" else 2e-2)
    assert (a - b).abs().max() <= tol * max(1.0, float(b.abs().max())), f"{what}: {float((a - b).abs().max()):.3e}"


def _sequences(lens, slots, dev):
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    return i32(starts), i32(slots), starts


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,d,dv", [(3, 16, 24), (2, 48, 8), (1, 130, 64), (4, 64, 128)])
def test_gated_linear_attention_scan_kernel(heads, d, dv, dtype):
    """Whole sequences and long portions in chunks, several sequences in slots of their own, a state carried over two steps."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(heads * d + dv)
    lens, slots = [200, 1, 70, 129], [2, 0, 3, 1]
    q_start, slot_t, starts = _sequences(lens, slots, dev)
    T = starts[-1]
    width = 2 * heads * d + heads * dv
    state = (0.1 * torch.randn(5, heads * d * dv + 3)).to(dev)
    for step in range(2):
        qkv = (0.5 * torch.randn(T, width)).to(dev, dt)
        za = (1.5 + torch.randn(T, heads * d + 4)).to(dev)
        got_state, ref_state = state.clone(), state.clone()
        got = torch.zeros(T, heads * dv, device=dev)
        ref = torch.zeros(T, heads * dv, device=dev)
        chunks = K.ScanChunks(starts, slots, dev)
        assert chunks.count > len(lens)
        K.gla_scan(qkv, 0, heads * d, 2 * heads * d, za, 4, 3.0, got_state, q_start, slot_t, got, heads, d, dv, chunks=chunks)
        R.gla_scan(qkv, 0, heads * d, 2 * heads * d, za, 4, 3.0, ref_state, q_start, slot_t, ref, heads, d, dv)
        _close(got, ref, dtype, "outputs in chunks", 1e-4)
        _close(got_state, ref_state, dtype, "states after chunks", 1e-4)
        one_state, one = state.clone(), torch.zeros(T, heads * dv, device=dev)
        K.gla_scan(qkv, 0, heads * d, 2 * heads * d, za, 4, 3.0, one_state, q_start, slot_t, one, heads, d, dv)
        _close(one, ref, dtype, "outputs in one piece", 1e-4)
        _close(one_state, ref_state, dtype, "states in one piece", 1e-4)
        assert torch.equal(one_state[4], state[4]) and torch.equal(one_state[:, -3:], state[:, -3:])       # nobody's slot, nobody's columns
        state = ref_state


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
# states of up to 64 elements run with a channel per thread (rows of 4, 8, 16, 32 and 64 registers), larger ones with a
# warp per eight channels: sizes that fill a row exactly, that leave part of it empty, and blocks of channels with a ragged end
@pytest.mark.parametrize("inner,N,rank", [(40, 12, 3), (8, 1, 1), (70, 33, 5), (256, 16, 8), (24, 130, 2), (200, 32, 2), (130, 64, 4), (33, 5, 1),
                                          (16, 65, 1)])
def test_selective_scan_with_a_state_row_per_channel_kernel(inner, N, rank, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(inner + N)
    lens, slots = [150, 1, 64, 131], [1, 3, 0, 2]
    q_start, slot_t, starts = _sequences(lens, slots, dev)
    T = starts[-1]
    state = (0.1 * torch.randn(5, inner * N + 2 * inner)).to(dev)
    A_log, D = (0.5 * torch.randn(inner, N)).to(dev), (1.0 + 0.2 * torch.randn(inner)).to(dev)
    for step in range(2):
        xz = (0.7 * torch.randn(T, 2 * inner)).to(dev, dt)
        low = (0.7 * torch.randn(T, rank + 2 * N)).to(dev, dt)
        dt32 = (-1.0 + torch.randn(T, inner)).to(dev)
        outs = []
        for how in ("chunks", "whole", "plain"):
            st, y = state.clone(), torch.zeros(T, inner, dtype=dt, device=dev)
            if how == "plain":
                R.channel_scan(xz, 0, low, rank, rank + N, dt32, xz, inner, A_log, D, st, q_start, slot_t, y)
            else:
                K.channel_scan(xz, 0, low, rank, rank + N, dt32, xz, inner, A_log, D, st, q_start, slot_t, y,
                               chunks=K.ScanChunks(starts, slots, dev) if how == "chunks" else None)
            outs.append((st, y))
        for (st, y), how in zip(outs[:2], ("chunks", "whole")):
            _close(y, outs[2][1], dtype, f"outputs ({how})", 1e-4 if dtype == "float32" else 2e-2)
            _close(st, outs[2][0], dtype, f"states ({how})", 1e-4)
            assert torch.equal(st[4], state[4]) and torch.equal(st[:, inner * N:], state[:, inner * N:])
        state = outs[2][0]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,groups,size", [(37, 3, 24), (9, 12, 128), (5, 2, 512), (5, 2, 513), (3, 1, 1200), (70, 1, 1), (6, 5, 300), (11, 7, 6)])
def test_gated_norm_kernel_in_short_and_long_groups(T, groups, size, dtype):
    """Groups of up to 512 elements are normed by a warp each, longer ones by a block: both against the plain reference,
    with the gate before the norm and (as a sigmoid or a silu) after it."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(T + size)
    n = groups * size
    y32 = torch.randn(T, n, device=dev) * 3.0
    w = (1.0 + 0.3 * torch.randn(n, device=dev))
    # the gate at a column and in rows that are multiples of four elements (loads of four at a time) and that are not
    for pad, col in ((12, 8), (11, 5)):
        gate = torch.randn(T, n + pad, device=dev).to(dt)
        for first, act in ((True, "sigmoid"), (False, "sigmoid"), (False, "silu")):
            a, b = (torch.empty(T, n, device=dev, dtype=dt) for _ in range(2))
            K.gated_rmsnorm(y32, gate, col, w, 1e-5, groups, first, a, gate_act=act)
            R.gated_rmsnorm(y32, gate, col, w, 1e-5, groups, first, b, gate_act=act)
            _close(a, b, dtype, f"gated norm, gate first {first}, {act}, gate at column {col}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_embedding_kernel_carries_the_previous_token_across_steps(dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(3)
    buckets, H, vocab = 11, 40, 29
    table = torch.randn(buckets + 1, H).to(dev, dt)
    seqs = {0: random_tokens(30, vocab, 1), 2: random_tokens(30, vocab, 2), 3: random_tokens(30, vocab, 3)}
    fed = {s: 0 for s in seqs}
    st_a, st_b = torch.zeros(5, 1, dtype=torch.int32, device=dev), torch.zeros(5, 1, dtype=torch.int32, device=dev)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    for portions in ([(0, 1), (2, 5), (3, 2)], [(2, 1), (0, 7)], [(3, 9), (0, 1), (2, 1)], [(0, 2), (3, 1)]):
        ids, pos, seq, starts, slots, want = [], [], [], [0], [], []
        for k, (s, n) in enumerate(portions):
            ids += seqs[s][fed[s]:fed[s] + n]
            pos += list(range(fed[s], fed[s] + n))
            # the rule itself: the first token takes the last row, every other one the row of (previous, current)
            want += [buckets if t == 0 else (seqs[s][t - 1] * 31 + seqs[s][t] * 7) % buckets for t in range(fed[s], fed[s] + n)]
            seq += [k] * n
            starts.append(len(ids))
            slots.append(s)
            fed[s] += n
        x0 = torch.randn(len(ids), H, device=dev)
        xa, xb = x0.clone(), x0.clone()
        K.add_pair_rows(xa, table, i32(ids), i32(pos), i32(starts), i32(seq), i32(slots), st_a, 31, 7)
        R.add_pair_rows(xb, table, i32(ids), i32(pos), i32(starts), i32(seq), i32(slots), st_b, 31, 7)
        _close(xa, xb, "float32", "rows added")
        _close(xa - x0, table.float()[torch.tensor(want, device=dev)], "float32", "the rows of the rule", 1e-5)
        assert torch.equal(st_a, st_b)
    assert [int(st_a[s, 0]) for s in (0, 2, 3)] == [seqs[s][fed[s] - 1] for s in (0, 2, 3)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_over_the_whole_projection_rotation_and_cache_write_kernel(dtype):
    """Keys and values of their own, and queries alone written into wider rows."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(9)
    nh, nkv, dh, real, T, page = 6, 2, 32, 24, 37, 16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    pos = i32(list(range(5, 5 + T)))
    slot_map = i32([(3 + (5 + t) // page) * page + (5 + t) % page for t in range(T)])
    denom = torch.tensor([3.0 ** j for j in range(4)], device=dev)
    for nkv_now in (nkv, 0):
        N = (nh + 2 * nkv_now) * dh
        proj = torch.randn(T, N).to(dev, dt)
        qn, kn = (1.0 + 0.2 * torch.randn(nh * dh)).to(dev), (1.0 + 0.2 * torch.randn(nkv * dh)).to(dev)
        rinv_a, rinv_b = torch.empty(T, 2, device=dev), torch.empty(T, 2, device=dev)
        ranges = [(0, nh * dh, nh * real)] + ([(nh * dh, nkv * dh, nkv * real)] if nkv_now else [])
        K.row_rinv(proj, ranges, 1e-5, rinv_a)
        R.row_rinv(proj, ranges, 1e-5, rinv_b)
        _close(rinv_a, rinv_b, "float32", "factors")
        outs = []
        for F, rinv in ((K, rinv_a), (R, rinv_b)):
            kc, vc = torch.zeros(8, nkv, page, dh, dtype=dt, device=dev), torch.zeros(8, nkv, dh, page, dtype=dt, device=dev)
            out = torch.zeros(T, (nh + 2 * nkv) * dh, dtype=dt, device=dev)
            F.conv_norm_rope_kv(proj, out, None, None, 0, i32([0, T]), i32([0] * T), i32([0]), qn, kn if nkv_now else None, 1e-5, real, pos, denom, 8,
                                slot_map, kc, vc, nh, nkv_now, dh, write=bool(nkv_now), row_rinv=rinv)
            outs.append((out[:, :nh * dh], kc, vc))
        for a, b, what in zip(outs[0], outs[1], ("queries", "keys", "values")):
            _close(a, b, dtype, f"{what} ({nkv_now} key heads)")
        assert bool(outs[0][1].abs().sum() > 0) == bool(nkv_now)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,ld,ranges", [(37, 56, [(8, 24, 20), (32, 16, 16)]), (19, 50, [(3, 20, 20), (25, 13, 11)]), (5, 4096, [(0, 3072, 3072), (3072, 512, 500)]),
                                         (9, 64, [(16, 48, 40)])])
def test_factors_of_a_norm_over_ranges_of_columns_kernel(T, ld, ranges, dtype):
    """Rows, ranges and columns that are multiples of a 16-byte load (a warp per token) and that are not (a block per token)."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(T + ld)
    x = (2.0 * torch.randn(T, ld, device=dev)).to(dt)
    a, b = (torch.zeros(T, 2, device=dev) for _ in range(2))
    K.row_rinv(x, ranges, 1e-5, a)
    R.row_rinv(x, ranges, 1e-5, b)
    _close(a[:, :len(ranges)], b[:, :len(ranges)], "float32", "factors", 1e-5)


@pytest.mark.gpu
def test_routing_by_the_softmax_over_the_chosen_logits_kernel():
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev = torch.device("cuda:0")
    torch.manual_seed(4)
    for E, top in ((5, 2), (1, 1), (70, 4), (16, 16)):
        logits = (3.0 * torch.randn(33, E)).to(dev)
        logits[0, 0] = -1e30                                   # a very low logit is still a logit
        a_ids, b_ids = torch.empty(33, top, dtype=torch.int32, device=dev), torch.empty(33, top, dtype=torch.int32, device=dev)
        a_w, b_w = torch.empty(33, top, device=dev), torch.empty(33, top, device=dev)
        K.moe_route(logits, top, a_ids, a_w, scoring="softmax_chosen")
        R.moe_route(logits, top, b_ids, b_w, scoring="softmax_chosen")
        assert torch.equal(a_ids, b_ids)
        _close(a_w, b_w, "float32", f"weights of {top} of {E}")
        assert (a_w.sum(-1) - 1.0).abs().max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [48, 100, 4096, 9000])
def test_the_stream_as_it_is_in_the_run_dtype_behind_a_norm_on_the_output(H, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(H)
    x = torch.randn(9, H, device=dev)
    y = torch.randn(9, H).to(dev, dt)
    w = (0.7 * (1.0 + 0.2 * torch.randn(H))).to(dev)
    xa, xb = x.clone(), x.clone()
    oa, ob = torch.empty(9, H, dtype=dt, device=dev), torch.empty(9, H, dtype=dt, device=dev)
    K.norm_add_norm(xa, y, (w, False, 1e-5), (None, False, 0.0), oa)
    R.norm_add_norm(xb, y, (w, False, 1e-5), (None, False, 0.0), ob)
    _close(xa, xb, "float32", "stream")
    _close(oa, ob, dtype, "the stream in the run dtype")
    assert torch.equal(oa.float(), xa.to(dt).float())
