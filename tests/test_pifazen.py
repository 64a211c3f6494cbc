"""The Pifazen decoder through the engine against the plain implementation (tests/plain_pifazen.py).

Small configurations of their own sizes and random weights, made here.  On a GPU the engine runs its CUDA kernels in
float32 and bfloat16; without one the same tests run the host-side logic (configuration, loader, cache manager with
pages and state slots, step function) over the kernels' plain references.  Covered: each mechanism alone; a prompt
whole, against its last tokens decoded one by one, against portions down to two tokens and one; unequal requests in one
batch against each alone, with pages and slots that are given back and used again; the first tokens of a sequence; a
token far back that only the recurrent state and a far key carry; long decoding from captured steps; layers that run on
another layer's tensors with a state of their own; a configuration of ones and sizes that are multiples of nothing;
greedy generation through the front end; configuration errors; random-weights mode; each new kernel against its plain
reference.
"""

from __future__ import annotations

import json
import math

import pytest
import torch

import plain_pifazen as P
from helpers import random_tokens

CUDA = torch.cuda.is_available()
DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]
DTYPES = ["float32", "bfloat16"]


def moe(experts=5, identity=1, top=3, count=3, keep=2, scale=1.5, ff=24, limit=1.5):
    router = {"experts": experts, "identity": identity, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def latent(heads=3, dim=16, rot=8, vdim=20, kv_rank=24, q_rank=20, base=5000.0, scale=0.21, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                      "rot": {"base": base, "dims": rot}}}


def latent2(heads=2, dim=8, rot=16, vdim=12, kv_rank=40, base=20000.0, scaling=(3.0, 64, 8.0, 2.0), scale=0.3, mlp=None):
    rot_cfg = {"base": base, "dims": rot}
    if scaling:
        rot_cfg["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot_cfg}}


def delta(heads=4, kv=2, dim=16, vdim=24, conv=3, mlp=None, weights_of=None):
    out = {"type": "channel_delta", "mlp": mlp, "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def config(layers, width=48, vocab=97, eps=1e-5):
    return {"architecture": "Pifazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# ranks of the low-rank maps of the delta layers (decays, output gate): config.json does not hold them, the tensors' shapes do
RANKS = {"delta_only": {0: (5, 7)}, "dense_only": {0: (4, 4)}, "mixed": {1: (6, 3), 3: (6, 3)}, "ones": {0: (1, 1)}, "odd": {1: (3, 5)},
         "wide": {1: (16, 24)}, "far": {0: (4, 4)}, "shared_later": {0: (4, 2), 2: (4, 2)}}

CONFIGS = {
    "delta_only": config([delta()]),
    "latent_only": config([latent()]),
    # (a latent and a rotated part that leave the attention head's last 8 elements empty)
    "latent2_only": config([latent2()]),
    "dense_only": config([delta(heads=2, kv=2, dim=8, vdim=8, conv=2, mlp=dense())]),
    "experts_only": config([latent(heads=2, dim=8, rot=4, vdim=8, kv_rank=12, q_rank=6, mlp=moe())]),
    # everything at once, no two sizes alike; layer 3 runs on layer 1's tensors with a state of its own
    "mixed": config([latent2(mlp=dense()), delta(mlp=moe()), latent(mlp=moe(experts=4, identity=0, top=2, count=2, keep=1, ff=16)),
                     delta(mlp=moe(), weights_of=1), latent2(heads=4, dim=12, rot=4, vdim=8, kv_rank=28, scaling=None, mlp=moe(experts=3, identity=3, top=6, count=0, ff=8))],
                    width=56, vocab=131),
    # a layer may name a later layer's tensors
    "shared_later": config([delta(heads=2, kv=1, dim=8, vdim=16, conv=4, mlp=dense(24), weights_of=2), latent(heads=2, dim=8, rot=4, vdim=8, kv_rank=12, q_rank=6),
                            delta(heads=2, kv=1, dim=8, vdim=16, conv=4, mlp=dense(24))], width=40, vocab=61),
    # one of everything
    "ones": config([delta(heads=1, kv=1, dim=4, vdim=4, conv=1, mlp=moe(experts=1, identity=0, top=1, count=1, keep=1, scale=1.0, ff=8)),
                    latent(heads=1, dim=4, rot=2, vdim=4, kv_rank=2, q_rank=1, scale=1.0, mlp=moe(experts=1, identity=1, top=1, count=2, keep=1, ff=8)),
                    latent2(heads=1, dim=2, rot=2, vdim=2, kv_rank=1, scaling=(1.0, 16, 4.0, 1.0), scale=1.0, mlp=dense(8))], width=16, vocab=29),
    # sizes that are multiples of nothing
    "odd": config([latent(heads=3, dim=12, rot=6, vdim=10, kv_rank=10, q_rank=7, mlp=dense(22)),
                   delta(heads=6, kv=2, dim=12, vdim=20, conv=2, mlp=moe(experts=7, identity=2, top=2, count=3, keep=2, ff=10)),
                   latent2(heads=5, dim=6, rot=10, vdim=18, kv_rank=18, mlp=None)], width=36, vocab=83),
    # sizes of a real model's layers: attention heads of 128 over the latent, key channels of 64, tiles of experts' rows
    "wide": config([latent(heads=4, dim=64, rot=32, vdim=64, kv_rank=96, q_rank=128, scale=0.1, mlp=dense(512)),
                    delta(heads=4, kv=2, dim=64, vdim=64, conv=4, mlp=moe(experts=6, identity=2, top=3, count=4, keep=3, ff=128)),
                    latent2(heads=4, dim=32, rot=16, vdim=64, kv_rank=48, scale=0.12, mlp=moe(experts=8, identity=0, top=2, count=2, keep=1, ff=128))],
                   width=256, vocab=512),
    # a state that forgets slowly (see make_weights) and full attention: a token far back still moves the last logits
    "far": config([delta(heads=2, kv=2, dim=16, vdim=16, conv=2), latent(heads=2, dim=8, rot=8, vdim=8, kv_rank=16, q_rank=8, scale=0.25)], width=32, vocab=41),
}


def with_ranks(name, cfg):
    """config.json with the ranks written into it, for the declared tensors (the plain side reads shapes only)."""
    cfg = json.loads(json.dumps(cfg))
    for i, (a, g) in RANKS.get(name, {}).items():
        cfg["layers"][i]["mixer"].update(decay_rank=a, gate_rank=g)
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
        if n == "head":
            continue                                  # the design has no head of its own: the logits come off the embedding table
        r = torch.randn(shape, generator=g)
        last = n.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2") or n == "final.norm":
            out[n] = 0.2 * r                                          # stored around zero, applied as 1 + w
        elif last in ("ls1", "ls2") or n.endswith("dq.norm") or n.endswith("dkv.norm") or n.endswith("mix.norm"):
            out[n] = 1.0 + 0.2 * r
        elif last == "dt_bias":
            out[n] = (-6.0 if name == "far" else -1.0) + 0.5 * r          # "far": decays near one, the state forgets slowly
        elif last == "A_log":
            out[n] = 0.5 * r - (2.0 if name == "far" else 0.5)
        elif last == "act":
            out[n] = torch.tensor([0.6, 0.3, 0.2, 0.1]) + 0.1 * r
        elif last == "correction":
            out[n] = 0.08 * r
        elif last == "b" and n.split(".")[-2] in ("up", "down"):
            out[n] = 0.3 * r
        elif last == "conv":
            out[n] = 0.6 * r
        elif last == "router":
            out[n] = r * (3.0 / math.sqrt(shape[-1]))
        elif n == "embed":
            out[n] = r
        else:
            out[n] = r * (1.5 / math.sqrt(shape[-1]))
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from litinfer_b200.weights.safetensors_io import write_file

    out = {}
    for k, (name, cfg) in enumerate(CONFIGS.items()):
        d = tmp_path_factory.mktemp("pifazen_" + name)
        w = make_weights(name, 311 + k)
        (d / "config.json").write_text(json.dumps(cfg))           # without the ranks: the engine reads them off the shapes
        write_file(d / "model.safetensors", w)
        out[name] = (d, cfg, w)
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
    # bfloat16: activations are rounded to 8 bits at a dozen places a layer.  A row may be unlucky, and a token whose
    # choice scores lie within that rounding of each other may go to another expert than in the plain model; most rows may
    # not (a wrong key or a lost state moves every row behind it by tens of percent)
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
@pytest.mark.parametrize("name", ["delta_only", "latent_only", "latent2_only", "dense_only", "experts_only", "ones", "shared_later"])
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
    # portions of two tokens from the start: the state and the convolution's inputs cross every step
    for i in range(10):
        run.step([("c", toks, 2)])
    assert_close(run.logits("c"), ref[:20], dtype, f"{name} in twos")


@pytest.mark.parametrize("device", DEVICES)
def test_the_residual_stream_after_every_layer(device, folders, request):
    """Float32, layer by layer: the stream after each layer run against the plain model's."""
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
    n = 300 if device == "cuda" else 110
    toks = random_tokens(n, cfg["vocab"], 11)
    ref = oracle("mixed", cfg, w, toks, dtype)
    run = Run(folder, dtype, dev, 320)
    run.step([("whole", toks, n)], end=["whole"])
    assert_close(run.logits("whole"), ref, dtype, "whole")
    # most of it at once, then token by token across page borders (16)
    run.step([("tail", toks, n - 50)])
    for i in range(50):
        run.step([("tail", toks, 1)], end=["tail"] if i == 49 else [])
    assert_close(run.logits("tail"), ref, dtype, "decoded")
    # portions of changing size, down to two tokens and one; the first token alone
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
    """Sizes that are multiples of nothing, and sizes of a real model's layers (on a GPU: the tensor-core attention over a
    head of 128, key channels of 64, tiles of experts' rows): a prompt whole, its end decoded, and in portions."""
    dev = use_device(device, request)
    folder, cfg, w = folders[name]
    n = 330 if device == "cuda" else 50
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
def test_a_token_far_back_reaches_the_last_logits_through_the_state_and_a_far_key(device, folders, request):
    """Two prompts that differ in their first token only.  With decays near one and full attention the last logits still
    differ, in the plain model and in the engine alike, whole and decoded one by one."""
    dev = use_device(device, request)
    folder, cfg, w = folders["far"]
    n = 260 if device == "cuda" else 120
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


def _weights_with_one_key_that_stands_out(cfg, w, hot_token):
    """Latent attention alone, weights changed by hand so that one token's key draws every later query: residual channel 0
    carries a constant that every token's query latent passes on to element 0 of each head's query, residual channel 1 is
    zero but for ``hot_token``, whose key latent passes it on to element 0 of each head's key."""
    w = {k: v.clone() for k, v in w.items()}
    m = cfg["layers"][0]["mixer"]
    H, d, dr = m["heads"], m["dim"], m["rot_dim"]
    w["embed"][:, 0] = 3.0
    w["embed"][:, 1] = 0.0
    w["embed"][hot_token, 1] = 6.0
    w["l0.norm1"][:2] = 0.0
    for name in ("l0.mix.dq", "l0.mix.dkv", "l0.mix.g"):
        w[name][:, :2] = 0.0                       # nothing else reads the two channels
    w["l0.mix.dq"][0] = 0.0
    w["l0.mix.dq"][0, 0] = 1.0                     # query latent 0 = the constant
    w["l0.mix.dkv"][0] = 0.0
    w["l0.mix.dkv"][0, 1] = 1.0                    # key/value latent 0 = the hot token's mark
    w["l0.mix.dq.norm"][0] = 1.0
    w["l0.mix.dkv.norm"][0] = 1.0
    for h in range(H):
        w["l0.mix.uq"][h * (d + dr)] = 0.0
        w["l0.mix.uq"][h * (d + dr), 0] = 8.0      # element 0 of every head's query
        w["l0.mix.uk"][h * d] = 0.0
        w["l0.mix.uk"][h * d, 0] = 8.0             # element 0 of every head's key
    w["l0.mix.uq"][:, 0] = torch.where(torch.arange(w["l0.mix.uq"].shape[0]) % (d + dr) == 0, w["l0.mix.uq"][:, 0], torch.zeros(()))
    w["l0.mix.uk"][:, 0] = torch.where(torch.arange(w["l0.mix.uk"].shape[0]) % d == 0, w["l0.mix.uk"][:, 0], torch.zeros(()))
    w["l0.mix.uv"][:, 0] = 2.0                     # and its value is unmistakable
    return w


@pytest.mark.parametrize("device", DEVICES)
def test_a_far_latent_key_with_one_score_made_to_stand_out(device, tmp_path, request):
    """Model level, latent attention alone, float32.  Random weights would bury one far key among hundreds, so the weights
    are made by hand (see above): the marked token's score stands out by tens of units for every later query, wherever it
    lies (the first place, a page's last and first place, far back, just before the decoded tokens).  Moving the mark by one
    place must move the logits of exactly the queries between the two places, in the plain model and in the engine alike, in
    a prompt's portion and in tokens decoded one by one."""
    from litinfer_b200.weights.safetensors_io import write_file

    dev = use_device(device, request)
    cfg = CONFIGS["latent_only"]
    hot_token = cfg["vocab"] - 1
    w = _weights_with_one_key_that_stands_out(cfg, make_weights("latent_only", 900), hot_token)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_file(tmp_path / "model.safetensors", w)
    w64 = {k: v.double() for k, v in w.items()}
    n = 200 if device == "cuda" else 70
    base = [t if t != hot_token else 0 for t in random_tokens(n, cfg["vocab"], 77)]
    for hot in (0, 15, 16, n // 2, n - 8):
        toks = list(base)
        toks[hot] = hot_token
        ref = P.forward(cfg, w64, toks).float()
        plain = P.forward(cfg, w64, base).float()
        moved = (ref - plain).abs().max(dim=-1).values
        assert float(moved[:hot].max() if hot else 0.0) < 1e-9 and float(moved[hot:].min()) > 0.5, f"mark at {hot}: the plain model does not see it as made"
        run = Run(tmp_path, "float32", dev, 256, graphs=False)
        run.step([("a", toks, n - 12)])
        for i in range(12):
            run.step([("a", toks, 1)], end=["a"] if i == 11 else [])
        assert_close(run.logits("a"), ref, "float32", f"mark at {hot}")
        # in portions that end right at the mark and right behind it
        cuts = [c for c in (hot, hot + 1) if 0 < c < n]
        at = 0
        for c in cuts + [n]:
            if c > at:
                run.step([("b", toks, c - at)], end=["b"] if c == n else [])
                at = c
        assert_close(run.logits("b"), ref, "float32", f"mark at {hot}, portions cut around it")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_captured_steps(dtype, folders):
    """300 tokens one by one (steps replayed from a captured graph: states, convolution inputs and pages moving on)
    against the prompt whole."""
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

    cfg = with_ranks("mixed", CONFIGS["mixed"])
    spec = config_from_dict(cfg).to_model_spec()
    assert spec.architecture == "Pifazen" and spec.tie_word_embeddings
    # the layer that runs on another's tensors is a schedule entry that names that layer's block again
    assert [e.block for e in spec.schedule] == [0, 1, 2, 1, 3] and len(spec.blocks) == 4
    assert [b.parts["mixer"].kind for b in spec.blocks] == ["latent_attention", "gated_delta_rule", "latent_attention", "latent_attention"]
    first = spec.blocks[0].parts["mixer"]
    assert first["q_rank"] is None and first["gate"] == "head" and first["position"]["scaling"]["kind"] == "yarn"
    assert spec.blocks[2].parts["mixer"]["gate"] == "element" and spec.blocks[2].parts["mixer"]["position"]["pairing"] == "interleaved"
    ff = spec.blocks[1].parts["feed_forward"]
    assert (ff["experts"], ff["identity"], ff["groups"], ff["keep_groups"], ff["top"]) == (5, 1, 3, 2, 3)
    assert spec.blocks[1].parts["mixer"]["decay_rank"] == 6 and spec.blocks[1].parts["mixer_post_norm"].kind == "channel_scale"

    def broken(change):
        c = json.loads(json.dumps(cfg))
        change(c)
        with pytest.raises(ConfigError):
            config_from_dict(c)

    broken(lambda c: c["layers"][0].update(type="attention"))
    broken(lambda c: c["layers"][0]["mlp"].update(kind="glu"))
    broken(lambda c: c["layers"][3].update(weights_of=3))
    broken(lambda c: (c["layers"][3].update(weights_of=1), c["layers"][1].update(weights_of=3)))       # a circle
    # a layer may name a layer that names another: it runs on the tensors at the end of that chain
    chain = json.loads(json.dumps(cfg))
    chain["layers"].append(dict(chain["layers"][3], weights_of=3))
    assert [e.block for e in config_from_dict(chain).to_model_spec().schedule] == [0, 1, 2, 1, 3, 1]
    broken(lambda c: c["layers"][3].update(weights_of=0))                       # another type than its own
    broken(lambda c: c["layers"][3]["mixer"].update(heads=8))                   # other sizes than the layer it names
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))             # more than the kept groups hold
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=4))  # 6 outputs do not form 4 groups
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6))             # the whole rotated part is rotated
    broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    broken(lambda c: c["norm"].update(eps=0.0))
    broken(lambda c: c["layers"][0]["mixer"].pop("scale"))


def test_random_weights_and_a_written_folder(tmp_path, cpu_kernels):
    """Random-weights mode knows the design's tensors; a folder written from it is read back through the registry, with
    the ranks taken from the tensors' shapes."""
    from litinfer_b200.config import load_config
    from litinfer_b200.models import DecoderModel
    from litinfer_b200.weights import write_model_folder

    cfg = with_ranks("mixed", CONFIGS["mixed"])
    write_model_folder(tmp_path, cfg, seed=5, store_dtype="float32")
    plain = json.loads((tmp_path / "config.json").read_text())
    for layer in plain["layers"]:
        layer["mixer"].pop("decay_rank", None)
        layer["mixer"].pop("gate_rank", None)
    (tmp_path / "config.json").write_text(json.dumps(plain))
    spec = load_config(tmp_path).to_model_spec()
    assert spec.blocks[1].parts["mixer"]["decay_rank"] == 6 and spec.blocks[1].parts["mixer"]["gate_rank"] == 3
    model = DecoderModel.from_dir(tmp_path, "float32", torch.device("cpu"))
    from litinfer_b200.engine.replay import Replayer

    rp = Replayer(model, 64, max_live=2, use_graphs=False)
    logits = rp.step({"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3, 4, 5], "want": [4]}], "end": ["a"]})
    assert logits.shape == (1, cfg["vocab"]) and torch.isfinite(logits).all() and float(logits.std()) > 0


# ---------------------------------------------------------------------------------------------
# the new kernels, each against its plain reference
# ---------------------------------------------------------------------------------------------

def _dt(dtype):
    return torch.float32 if dtype == "float32" else torch.bfloat16


def _close(a, b, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype == "float32" else 2e-2)
    scale = max(1.0, float(b.float().abs().max()))
    assert float((a.float() - b.float()).abs().max()) <= tol * scale, f"{what}: {float((a.float() - b.float()).abs().max()):.3e} (scale {scale:.2f})"


def _sequences(lens, slots, dev):
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    return torch.tensor(starts, dtype=torch.int32, device=dev), torch.tensor(slots, dtype=torch.int32, device=dev)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv,d,dv,taps", [(2, 2, 16, 8, 3), (4, 2, 32, 40, 4), (3, 1, 20, 17, 1), (2, 1, 64, 64, 2), (2, 2, 128, 72, 4), (1, 1, 130, 9, 3)])
def test_gated_delta_rule_kernels(heads, kv, d, dv, taps, dtype):
    """The kernel that prepares a token (convolution, unit vectors, decays, beta) and the walk over the state, each against
    its reference: shared key heads, an empty sequence, slots and tails of slots that nobody owns, a portion against its
    tokens one by one (where the convolution's state moves on inside the first kernel)."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(heads * 100 + d)
    lens, slots = [37, 1, 0, 18], [2, 0, 3, 1]
    T = sum(lens)
    q_start, sl = _sequences(lens, slots, dev)
    seq = torch.tensor([s for s, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device=dev)
    C, S_el, DP = 2 * kv * d + heads * dv, heads * d * dv, K.delta_row_elements(d)
    proj = torch.randn(T, 3 + C + heads + 5, device=dev).to(dt)
    conv_w = (0.6 * torch.randn(C, taps, device=dev)).contiguous()
    za = (torch.randn(T, heads * d + 2, device=dev) - 2.0).contiguous()
    A_log = (0.5 * torch.randn(heads, device=dev) - 0.5).contiguous()
    state = 0.3 * torch.randn(5, S_el + (taps - 1) * C + 11, device=dev)

    def buffers(n):
        return (torch.empty(n, kv, 2 * DP + 4, device=dev), torch.empty(n, heads, DP + 4, device=dev), torch.empty(n, heads * dv, device=dev))

    got, ref = buffers(T), buffers(T)
    K.delta_prepare(proj, 3, 3 + C + 1, conv_w, state, S_el, q_start, seq, sl, za, 1, A_log, *got, heads, kv, d, dv)
    R.delta_prepare(proj, 3, 3 + C + 1, conv_w, state, S_el, q_start, seq, sl, za, 1, A_log, *ref, heads, kv, d, dv)
    for a, b, what in zip(got, ref, ("q, k and their product", "decays and beta", "values")):
        _close(a[..., :-3] if a.dim() == 3 else a, b[..., :-3] if b.dim() == 3 else b, "float32", what, 1e-5)
    ref_state, out, want = state.clone(), torch.zeros(T, heads * dv, device=dev), torch.zeros(T, heads * dv, device=dev)
    state0 = state.clone()
    K.delta_scan(*got, state, q_start, sl, out, heads, kv, d, dv)
    R.delta_scan(*ref, ref_state, q_start, sl, want, heads, kv, d, dv)
    _close(out, want, "float32", "outputs", 1e-4)
    _close(state, ref_state, "float32", "states", 1e-4)
    assert torch.equal(state[4], ref_state[4]) and torch.equal(state[:, S_el:], ref_state[:, S_el:]), "a slot or the tail of a slot that no sequence owns was touched"
    # a warp of the walk holds two, four or eight columns, by the size of the launch: the same bits whichever it is
    import ctypes
    try:
        for columns in (2, 4, 8):
            K.library().li_delta_force_columns(ctypes.c_int(columns))
            again_state, again = state0.clone(), torch.zeros_like(out)
            K.delta_scan(*got, again_state, q_start, sl, again, heads, kv, d, dv)
            assert torch.equal(again, out) and torch.equal(again_state, state), f"{columns} columns a warp"
    finally:
        K.library().li_delta_force_columns(ctypes.c_int(0))
    # the first sequence again, one token at a time, from the state it had: the same outputs, and the convolution's inputs kept
    one_state, outs = ref_state.clone().copy_(0.3 * torch.randn_like(state)), torch.zeros(37, heads * dv, device=dev)
    whole_state, whole = one_state.clone(), torch.zeros(37, heads * dv, device=dev)
    first = buffers(37)
    qs37, sl1 = q_start[:2].contiguous(), sl[:1].contiguous()
    K.delta_prepare(proj[:37].contiguous(), 3, 3 + C + 1, conv_w, whole_state, S_el, qs37, seq[:37].contiguous(), sl1, za[:37].contiguous(), 1, A_log, *first, heads, kv, d, dv)
    if taps > 1:
        K.conv_state_shift(proj[:37].contiguous(), 3, C, taps, whole_state, S_el, qs37, sl1)
    K.delta_scan(*first, whole_state, qs37, sl1, whole, heads, kv, d, dv)
    qs1, seq1 = torch.tensor([0, 1], dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
    for t in range(37):
        step = buffers(1)
        K.delta_prepare(proj[t:t + 1].contiguous(), 3, 3 + C + 1, conv_w, one_state, S_el, qs1, seq1, sl1, za[t:t + 1].contiguous(), 1, A_log, *step, heads, kv, d, dv,
                        shift=True)
        K.delta_scan(*step, one_state, qs1, sl1, outs[t:t + 1], heads, kv, d, dv)
    _close(outs, whole, "float32", "token by token against the portion", 1e-4)
    _close(one_state, whole_state, "float32", "states and convolution inputs token by token", 1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,n", [(5, 24), (3, 1000), (2, 9000), (2, 20000)])
def test_polynorm_kernel(T, n, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(n)
    z = (1.3 * torch.randn(T, n, device=dev)).to(dt)
    coef = torch.tensor([0.7, -0.4, 0.25, 0.1], device=dev)
    out, ref = torch.empty_like(z), torch.empty_like(z)
    K.polynorm(z, coef, 1e-5, out)
    R.polynorm(z, coef, 1e-5, ref)
    _close(out, ref, dtype, "polynorm")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_sigmoid_gate_kernel_per_element_and_per_head(dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(4)
    for n, group in ((60, 1), (60, 20), (7, 7)):
        x = torch.randn(9, n, device=dev).to(dt)
        gate = (2 * torch.randn(9, 70, device=dev)).to(dt)
        ref = x.clone()
        K.mul_sigmoid(x, gate, 5, group)
        R.mul_sigmoid(ref, gate, 5, group)
        _close(x, ref, dtype, f"gate in groups of {group}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,d,R_,dr,dl,interleaved,mag", [(3, 8, 24, 8, 32, True, 1.0), (2, 4, 40, 16, 64, True, 1.13), (1, 2, 1, 2, 16, False, 1.0), (4, 16, 10, 6, 16, True, 0.9)])
def test_latent_rotation_and_norm_kernel(nh, d, R_, dr, dl, interleaved, mag, dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    torch.manual_seed(nh + dl)
    T = 11
    low = torch.randn(T, 7 + R_ + dr + 3, device=dev).to(dt)
    q = torch.randn(T, nh * (d + dr) + 4, device=dev).to(dt)
    w = (1.0 + 0.2 * torch.randn(R_, device=dev)).contiguous()
    pos = torch.randint(0, 3000, (T,), dtype=torch.int32, device=dev)
    denom = torch.pow(torch.tensor(700.0), torch.arange(dr // 2) * 2.0 / dr).to(dev)
    out = torch.full((T, (nh + 2) * dl), 7.0, device=dev).to(dt)
    ref = out.clone()
    K.latent_rope_post(low, 7, 7 + R_, q, d, w, 1e-5, pos, denom, mag, interleaved, out, nh, R_, dr, dl)
    R.latent_rope_post(low, 7, 7 + R_, q, d, w, 1e-5, pos, denom, mag, interleaved, ref, nh, R_, dr, dl)
    _close(out, ref, dtype, "rows", 2e-3 if dtype == "float32" else 2e-2)            # (angles of thousands of radians in float32)
    got = out.view(T, nh + 2, dl)
    assert (got[:, :nh, :R_] == 7.0).all(), "the queries' first columns belong to the product before"
    assert (got[:, :, R_ + dr:] == 0).all() and (got[:, nh + 1, R_:] == 0).all()


@pytest.mark.gpu
def test_routing_over_all_outputs_with_groups_kernel():
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev = torch.device("cuda:0")
    for E, top, groups, keep, corr in ((12, 4, 4, 3, True), (6, 3, 3, 2, True), (5, 2, 1, 1, False), (1, 1, 1, 1, True), (64, 6, 8, 2, True), (40, 8, 5, 5, True)):
        torch.manual_seed(E)
        logits = (2 * torch.randn(300, E, device=dev)).contiguous()
        correction = (0.1 * torch.randn(E, device=dev)).contiguous() if corr else None
        ids, wt = torch.empty(300, top, dtype=torch.int32, device=dev), torch.empty(300, top, device=dev)
        rids, rwt = torch.empty_like(ids), torch.empty_like(wt)
        K.moe_route_grouped(logits, correction, top, groups, keep, 1.7, ids, wt)
        R.moe_route_grouped(logits, correction, top, groups, keep, 1.7, rids, rwt)
        same = (ids == rids).all(dim=1)
        assert same.float().mean() > 0.99, f"{E} outputs: {int((~same).sum())} tokens chose otherwise"
        assert (wt[same] - rwt[same]).abs().max() < 1e-5
        assert ((wt.sum(-1) - 1.7).abs() < 1e-4).all()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", DTYPES)
def test_a_factor_per_channel_behind_a_sublayer_kernel(dtype):
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev, dt = torch.device("cuda:0"), _dt(dtype)
    for H in (40, 36, 9000):
        torch.manual_seed(H)
        x = torch.randn(6, H, device=dev)
        y = torch.randn(6, H, device=dev).to(dt)
        ls, wn = (1 + 0.3 * torch.randn(H, device=dev)).contiguous(), (1 + 0.3 * torch.randn(H, device=dev)).contiguous()
        rx, out, ref = x.clone(), torch.empty(6, H, device=dev, dtype=dt), torch.empty(6, H, device=dev, dtype=dt)
        K.norm_add_norm(x, y, (ls, K.SCALE_ONLY, 0.0), (wn, False, 1e-5), out)
        R.norm_add_norm(rx, y, (ls, 2, 0.0), (wn, False, 1e-5), ref)
        _close(x, rx, "float32", f"stream of {H}", 1e-5)
        _close(out, ref, dtype, f"next norm of {H}")


@pytest.mark.gpu
@pytest.mark.parametrize("rows_per_token", [1, 40])
def test_experts_with_bounded_units_and_rows_of_no_expert(rows_per_token):
    """The grouped products with the bounded unit in their epilogue (few rows: the weight-streaming tiles; many: the tcgen05
    tiles of 128 rows): rows behind the last expert's run, the identity experts', pass untouched."""
    import kernel_refs as R
    from litinfer_b200 import kernels as K

    dev = torch.device("cuda:0")
    torch.manual_seed(rows_per_token)
    E, extra, top, W, F = 5, 2, 3, 64, 48
    T = 8 * rows_per_token
    ids = torch.randint(0, E + extra, (T, top), dtype=torch.int32, device=dev)
    pad = 128 if T * top >= 256 else 1
    Rr = K.sorted_rows(T * top, E + extra, pad)
    offsets, pair_at, place_of = (torch.empty(n, dtype=torch.int32, device=dev) for n in (E + extra + 1, Rr, T * top))
    tiles = torch.empty(Rr // pad, dtype=torch.int32, device=dev) if pad > 1 else None
    K.moe_sort(ids, E + extra, offsets, pair_at, place_of, pad, tiles, matrices=E)
    ro, rp_, rpl = torch.empty_like(offsets), torch.empty_like(pair_at), torch.empty_like(place_of)
    rt = torch.empty_like(tiles) if tiles is not None else None
    R.moe_sort(ids, E + extra, ro, rp_, rpl, pad, rt, matrices=E)
    assert torch.equal(offsets, ro) and torch.equal(pair_at, rp_) and torch.equal(place_of, rpl)
    if tiles is not None:
        assert torch.equal(tiles, rt) and int(tiles.max()) == E - 1
    h = torch.randn(T, W, device=dev).to(torch.bfloat16)
    rows = torch.empty(Rr, W, device=dev, dtype=torch.bfloat16)
    K.moe_gather(h, pair_at, None, top, rows)
    gate, up = (torch.randn(E, F, W, device=dev) / 8).to(torch.bfloat16), (torch.randn(E, F, W, device=dev) / 8).to(torch.bfloat16)
    gu = torch.stack([K.interleave_gate_up(gate[e].contiguous(), up[e].contiguous()) for e in range(E)]).contiguous()
    params = torch.tensor([1.2, 1.702], device=dev)
    act, ref = torch.full((Rr, F), 3.0, device=dev, dtype=torch.bfloat16), torch.full((Rr, F), 3.0, device=dev, dtype=torch.bfloat16)
    K.grouped_linear(rows, gu, act, offsets[:E + 1], tile_group=tiles, epilogue="glu_clamped", epilogue_params=params)
    R.grouped_linear(rows, gu, ref, offsets[:E + 1], tile_group=tiles, epilogue="glu_clamped", epilogue_params=params)
    lo = int(offsets[E])
    live = (pair_at[:lo] >= 0)
    _close(act[:lo][live], ref[:lo][live], "bfloat16", "activations")
    assert (act[lo:] == 3.0).all(), "rows of no expert were written"
    down = (torch.randn(E, W, F, device=dev) / 8).to(torch.bfloat16)
    before = rows.clone()
    K.grouped_linear(ref, down, rows, offsets[:E + 1], tile_group=tiles)
    assert torch.equal(rows[lo:], before[lo:]), "the identity experts' rows must stay the gathered input"
