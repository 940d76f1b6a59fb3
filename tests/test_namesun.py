"""Namesun in the engine against the plain implementation (tests/plain/namesun_plain.py).

Without a GPU the engine runs on the stand-in kernel namespace (tests/ref_ops.py), which
exercises configuration, weights, spec, parts, cache and state manager, batch builder,
scheduler and entry point.  With a GPU (-m gpu) the same checks run on the CUDA kernels in
float32 and bfloat16, plus each kernel alone against the plain statement of its op."""
import io
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from mini_inference_b200 import LLM, SamplingParams
from mini_inference_b200.config import ConfigError, load_config, resolve
from mini_inference_b200.config.namesun_config import NamesunConfig
from mini_inference_b200.engine.batch import StepEntry
from mini_inference_b200.engine.factory import load_model, make_runner
from mini_inference_b200.weights import write_random_model
from tests.plain import namesun_plain as plain
from tests.ref_ops import TorchRefOps

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def attn(heads, kv, dim, vdim, block=None, v_mix=False, scale=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else 1.7 * dim ** -0.5}
    if block:
        m["mask"] = {"size": block}
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": mlp}


def ret(heads, dim, vdim, decay, rot_dims=None, base=10000.0, mlp=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                           "rot": {"dims": dim if rot_dims is None else rot_dims, "base": base}}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(width, vocab, layers, mult=0.5, eps=1e-5):
    return {"architecture": "Namesun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}


# Small configurations that differ from one another in every size; none makes two sizes equal by accident.
CONFIGS = {
    # both mixers, blocks of 7 positions (edges inside every page and portion), three layers that blend values (the middle one
    # is the second of them), grouped and ungrouped routers, a layer without feed-forward
    "mix": (config(48, 131, [attn(6, 2, 8, 12, block=7, v_mix=True, mlp=moe(6, 2, 10, 1.5, groups=(3, 2), shared=(14, 0.8))),
                             ret(3, 8, 10, [0.5, 0.9, 0.99], rot_dims=4, mlp=dense(40)),
                             attn(4, 2, 16, 12, block=11, v_mix=True, mlp=moe(5, 3, 12, 3.0)),
                             attn(2, 2, 8, 12, v_mix=True), ret(2, 12, 6, [0.8, 0.97], mlp=dense(36))], mult=0.4), 4),
    # one query head per key head and one head in all; a block longer than any request; no layer blends values; one expert of one
    "ones": (config(40, 97, [ret(1, 16, 20, [0.93], rot_dims=16, base=100.0, mlp=moe(3, 1, 8, 0.7, groups=(3, 1))),
                             attn(1, 1, 24, 8, block=500, mlp=dense(56))], mult=1.0, eps=1e-6), 8),
    # blocks equal to the page size and to twice it; every group kept; top = all eligible experts; no shared expert
    "pages": (config(64, 150, [attn(4, 1, 16, 16, block=16, v_mix=True, mlp=moe(4, 4, 16, 2.5, groups=(2, 2))),
                               attn(8, 4, 8, 4, block=32, mlp=moe(8, 2, 8, 1.0, groups=(8, 3), shared=(24, 1.0))),
                               ret(4, 8, 16, [0.6, 0.9, 0.97, 0.999], rot_dims=2, base=1e6, mlp=None)], mult=0.25), 16),
    # key = value rows of 64 and of 128 entries on pages of 16: in bfloat16 on the GPU these reach the tensor-core prompt and decode
    # kernels, also in mixed batches; the third layer blends the first one's values
    "rows64": (config(64, 113, [attn(4, 2, 64, 64, block=24, v_mix=True, mlp=moe(4, 2, 64, 1.2, shared=(64, 1.5))),
                                ret(2, 16, 8, [0.9, 0.99], rot_dims=8, mlp=dense(48)),
                                attn(2, 2, 64, 64, block=50, v_mix=True, mlp=dense(72)), attn(2, 1, 128, 128, block=37)], mult=0.6), 16),
}
STD = 0.25


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (name, (cfg, page)) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("namesun_" + name))
        write_random_model(cfg, d, seed=20 + i, std=STD, norm_init="uniform")
        _perturb_corrections(d)
        out[name] = (d, cfg, page)
    return out


def _perturb_corrections(d):
    """The random-weights writer leaves the routers' corrections at zero; give them values that change the choice."""
    from mini_inference_b200.weights.safetensors_io import write_safetensors
    cfg, w = plain.load_model_dir(d)
    g = torch.Generator().manual_seed(7)
    for name in w:
        if name.endswith(".correction"):
            w[name] = (torch.randn(w[name].shape, generator=g) * 0.15).to(w[name].dtype)
    write_safetensors(os.path.join(d, "model.safetensors"), [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in w.items()])


def tokens(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_PLAIN = {}


def plain_logits(d, ids):
    if d not in _PLAIN:
        _PLAIN[d] = plain.load_model_dir(d)
    cfg, w = _PLAIN[d]
    return plain.forward_logits(cfg, w, ids).float()


def err(got, want):
    return ((got - want).abs().max() / want.abs().max()).item()


def assert_close(got, want, tol, what=""):
    """float32 (tol < 1e-2): every position within tol.  bfloat16: the rows that reach a router carry 8 mantissa bits, so where two
    experts' choice scores nearly tie, the choice can fall the other way than in the plain implementation, and that token (and,
    through cache and state, some later ones) then differs by more than rounding.  So: the median position within tol / 3 and at
    most one position in six beyond tol; what the mechanisms compute is pinned by the float32 runs and the kernels' own tests."""
    if tol < 1e-2:
        assert err(got, want) < tol, (what, err(got, want))
        return
    per = (got - want).abs().amax(-1) / want.abs().max()
    assert per.median().item() < tol / 3 and (per > tol).float().mean().item() <= 1 / 6, (what, per.median().item(), per.max().item())


def engine(d, page, pages, dtype="float32", device="cpu", max_seqs=4):
    _, model, _ = load_model(d, dtype, device)
    return make_runner(model, page, pages, max_seqs, ops=TorchRefOps() if device == "cpu" else None)


def feed(runner, key, ids, cuts):
    seq = runner.cache.admit(key)
    out, at = [], 0
    for n in cuts:
        out.append(runner.step([StepEntry(seq, ids[at:at + n], range(n))]).float().cpu())
        at += n
    assert at == len(ids)
    runner.cache.free(seq)
    return torch.cat(out)


def portions(n, rng, smallest=2, largest=9):
    cuts = []
    while n > 0:
        c = min(n, rng.randint(smallest, largest))
        if n - c == 1:
            c += 1
        cuts.append(c)
        n -= c
    return cuts


def check_cuts(runner, d, vocab, tol, n=61):
    """Whole prompt; most of it then the last 24 one by one; portions of 2..9 tokens; portions of two; from the first token
    one by one (long decoding: every state and cache row is written one token at a time, every block edge is crossed)."""
    ids = tokens(vocab, n, seed=3)
    want = plain_logits(d, ids)
    free = runner.cache.free_pages()
    assert_close(feed(runner, "w", ids, [n]), want, tol)
    assert_close(feed(runner, "d", ids, [n - 24] + [1] * 24), want, tol)
    assert_close(feed(runner, "p", ids, portions(n, random.Random(1))), want, tol)
    assert_close(feed(runner, "2", ids[:20], [2] * 10), want[:20], tol)
    assert_close(feed(runner, "1", ids, [1] * n), want, tol)
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == free


def check_mixed(make, d, vocab, page, tol, lens=(23, 9, 31, 17, 40, 12, 27, 36, 20, 33), seed=7):
    """Up to four live requests, portions of some beside single tokens of others, some left out of a step; the pool holds
    four of the longest requests and there are four state slots, so pages and slots are used again (both counted)."""
    rng = random.Random(seed)
    reqs = {f"r{i}": tokens(vocab, n, seed=100 + i) for i, n in enumerate(lens)}
    want = {k: plain_logits(d, v) for k, v in reqs.items()}
    pages = 4 * -(-max(lens) // page)
    runner = make(pages)
    takes, slot_uses = {}, {}
    for g in runner.cache.kv_groups:
        inner = g.pool.take
        def counted(inner=inner, gi=id(g)):
            pg = inner()
            takes[(gi, pg)] = takes.get((gi, pg), 0) + 1
            return pg
        g.pool.take = counted
    pending, live, got = list(reqs), {}, {k: [] for k in reqs}
    while pending or live:
        while pending and len(live) < 4:
            k = pending.pop(0)
            live[k] = [runner.cache.admit(k), 0]
            slot_uses[live[k][0].slot] = slot_uses.get(live[k][0].slot, 0) + 1
        entries, owners = [], []
        for k, (seq, at) in live.items():
            if rng.random() < 0.2 and len(live) > 1:
                continue
            left = len(reqs[k]) - at
            n = 1 if (at > 0 and rng.random() < 0.5) else min(left, rng.randint(2, 8))
            if left - n == 1:
                n = left
            entries.append(StepEntry(seq, reqs[k][at:at + n], range(n)))
            owners.append((k, n))
        if not entries:
            continue
        logits = runner.step(entries).float().cpu()
        row = 0
        for k, n in owners:
            got[k].append(logits[row:row + n])
            row += n
            live[k][1] += n
        for k in [k for k, (seq, at) in live.items() if at == len(reqs[k])]:
            runner.cache.free(live.pop(k)[0])
        runner.cache.check_invariants()
    for k in reqs:
        assert_close(torch.cat(got[k]), want[k], tol, k)
    assert runner.cache.free_pages() == pages
    assert len(slot_uses) <= 4 and max(slot_uses.values()) >= 2, "no state slot was used again"
    assert sum(n - 1 for n in takes.values()) * 3 >= sum(takes.values()), "too few pages were used again"


# ---------------------------------------------------------------- configuration, registry, spec, cache needs
def test_config_reads_every_key_and_refuses_what_is_missing():
    raw = CONFIGS["mix"][0]
    assert resolve(raw).name == "Namesun" and resolve({"architectures": ["Namesun"]}).name == "Namesun"
    cfg = NamesunConfig.from_dict(raw)
    assert NamesunConfig.from_dict(cfg.to_dict()) == cfg and cfg.residual_mult == 0.4
    assert cfg.layers[0].mlp.groups == (3, 2) and cfg.layers[0].mlp.shared == (14, 0.8) and cfg.layers[3].mlp is None
    assert cfg.layers[1].mixer_dict()["rot"] == {"base": 10000.0, "dims": 4} and cfg.layers[2].mixer_dict()["mask"] == {"size": 11}
    for path, msg in ((("norm",), "norm"), (("residual_mult",), "residual_mult"), (("layers", 1, "mixer", "decay"), "decay"),
                      (("layers", 1, "mixer", "rot"), "rot"), (("layers", 0, "mixer", "scale"), "scale"),
                      (("layers", 0, "mlp", "expert"), "expert"), (("layers", 0, "mlp", "router", "top"), "top"), (("vocab",), "vocab")):
        broken = json.loads(json.dumps(raw))
        node = broken
        for p in path[:-1]:
            node = node[p]
        del node[path[-1]]
        with pytest.raises(ConfigError, match=msg):
            NamesunConfig.from_dict(broken)
    for edit, msg in ((lambda c: c["layers"][0].update(type="window_attention"), "window_attention"),
                      (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
                      (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
                      (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
                      (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "conv")):
        bad = json.loads(json.dumps(raw))
        edit(bad)
        with pytest.raises(ConfigError, match=msg):
            NamesunConfig.from_dict(bad)


def test_spec_and_cache_needs(dirs):
    d, cfg, page = dirs["mix"]
    _, spec = load_config(d)
    assert spec.residual == "float32" and spec.embedding_norm is None
    roles = [spec.layers[i].part("mixer").get("value_mix") for i in range(5)]
    assert roles == ["source", None, "blend", "blend", None]
    assert spec.layers[3].block == "outnorm_mixer" and spec.layers[1].part("feed_forward").kind == "swiglu"
    runner = engine(d, page, 8)
    caches = runner.cache.layer_caches
    # value rows of 12 beside key rows of 8 and 16: pools of their own; layers 0 and 3 share a group (same sizes)
    assert caches[0].k.shape[-1] == 8 and caches[0].v.shape[-1] == 12 and caches[2].k.shape[-1] == 16
    assert caches[0].group == caches[3].group != caches[2].group
    assert caches[1].state.shape[1] == 3 * 8 * 10 and caches[4].state.shape[1] == 2 * 12 * 6
    d, cfg, page = dirs["pages"]
    runner = engine(d, page, 8)
    assert runner.cache.layer_caches[0].v.shape[-1] == 16                        # equal sizes: the two planes of one tensor
    assert runner.cache.bytes_per_token() == (1 * (16 + 16) + 4 * (8 + 4)) * 4


# ---------------------------------------------------------------- the plain functions on inputs whose answer is known
def test_plain_mechanisms_by_hand():
    f64 = torch.float64
    x = torch.tensor([[3.0, 4.0]], dtype=f64)
    assert torch.allclose(plain.rms(x, 0.0), x / (12.5 ** 0.5))
    # rotate-half: coordinate 0 pairs with 2 (dims = 4 of 5), coordinate 4 passes
    v = torch.tensor([[[1.0, 0.0, 0.0, 2.0, 9.0]]], dtype=f64)
    r = plain.rotate_half(v, torch.tensor([3]), 4, 100.0)
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    assert torch.allclose(r[0, 0], torch.tensor([math.cos(a0), -2 * math.sin(a1), math.sin(a0), 2 * math.cos(a1), 9.0], dtype=f64))
    # one key, score s: the weight is e^s / (1 + e^s), not 1
    w = {"q": torch.eye(2, dtype=f64), "k": torch.eye(2, dtype=f64), "v": torch.eye(2, dtype=f64), "o": torch.eye(2, dtype=f64)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5, "mask": {"size": 2}}
    h = torch.tensor([[1.0, 1.0], [2.0, 2.0], [1.0, -1.0]], dtype=f64)
    out, _ = plain.chunked_sink_attention(h, w, "", m, 0.0)
    s = 0.5 * 2.0                                                  # unit-RMS q and k of (1, 1): q . k = 2
    assert torch.allclose(out[0], h[0] * math.exp(s) / (1 + math.exp(s)))
    # position 2 opens a new block of two: it sees only itself
    assert torch.allclose(out[2], h[2] * math.exp(s) / (1 + math.exp(s)))
    # the router: groups (0,1) (2,3) (4,5); the correction lifts expert 5 into the choice, the weight stays its plain score
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    wr = {"router": torch.tensor([[0.0], [1.0], [2.0], [0.5], [0.1], [0.2]], dtype=f64), "correction": torch.tensor([0, 0, 0, 0, 0, 5.0], dtype=f64)}
    idx, wt = plain.route(torch.ones(1, 1, dtype=f64), wr, "", r)
    sm = torch.softmax(wr["router"][:, 0], 0)
    assert idx.tolist() == [[5, 4]] and torch.allclose(wt[0], sm[[5, 4]])
    # the expert: gate 5 -> 2 (limit), up -7 -> -2: y = 2 sigmoid(3.404) (-1)
    we = {"gate": torch.tensor([[5.0]], dtype=f64), "up": torch.tensor([[-7.0]], dtype=f64), "down": torch.tensor([[1.0]], dtype=f64)}
    y = plain.clamped_expert(torch.ones(1, 1, dtype=f64), we, "", 2.0)
    assert torch.allclose(y, torch.tensor([[-2.0 / (1 + math.exp(-3.404))]], dtype=f64))


# ---------------------------------------------------------------- each mechanism alone (one layer)
SINGLE = {
    "attention_blocks": config(32, 61, [attn(4, 2, 8, 6, block=5)]),
    "attention_whole": config(32, 61, [attn(3, 3, 8, 10)], mult=1.3),
    "attention_blend": config(32, 61, [attn(2, 1, 8, 6, block=9, v_mix=True), attn(4, 1, 16, 6, block=4, v_mix=True)]),
    "retention": config(36, 67, [ret(3, 8, 10, [0.3, 0.9, 0.999])]),
    "retention_part_rotated": config(36, 67, [ret(2, 12, 5, [0.7, 0.95], rot_dims=6, base=50.0)]),
    "retention_unrotated": config(36, 67, [ret(2, 6, 9, [0.85, 0.6], rot_dims=0)]),
    "dense": config(40, 71, [ret(1, 4, 4, [0.5], mlp=dense(52))]),
    "experts_grouped": config(40, 71, [ret(1, 4, 4, [0.5], mlp=moe(12, 3, 7, 0.9, groups=(4, 2), shared=(9, 2.0)))]),
    "experts_plain": config(40, 71, [ret(1, 4, 4, [0.5], mlp=moe(5, 2, 11, 4.0))]),
    # sizes that put every view of a fused product on an odd offset
    "attention_odd": config(27, 53, [attn(3, 1, 8, 5, block=3)]),
    "attention_odd_keys": config(27, 53, [attn(2, 2, 7, 3, block=6), attn(4, 1, 10, 9)]),
    # key and value rows of 64 entries: in bfloat16 on the GPU prompt portions take the tensor-core kernel
    "attention_rows64": config(48, 61, [attn(3, 1, 64, 64, block=40), attn(2, 2, 64, 64)]),
    "retention_odd": config(27, 53, [ret(3, 5, 7, [0.4, 0.8, 0.95], rot_dims=2)]),
    "experts_odd": config(27, 53, [ret(1, 3, 3, [0.5], rot_dims=2, mlp=moe(3, 2, 5, 1.1, groups=(3, 2), shared=(3, 0.5)))]),
}


def single_dir(tmp_path, name):
    d = write_random_model(SINGLE[name], str(tmp_path), seed=3, std=0.3, norm_init="uniform")
    _perturb_corrections(d)
    return d


@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name):
    cfg = SINGLE[name]
    d = single_dir(tmp_path, name)
    ids = tokens(cfg["vocab"], 37, seed=1)
    want = plain_logits(d, ids)
    c0, w = plain.load_model_dir(d)
    w = {k: v.double() for k, v in w.items()}
    bare = ((plain.rms(w["embed"][torch.tensor(ids)], c0["norm"]["eps"]) * w["final.norm"]) @ w["head"].T).float()
    assert err(bare, want) > 0.05                               # the layer matters
    runner = engine(d, 4, 16)
    assert err(feed(runner, "w", ids, [37]), want) < 2e-5
    assert err(feed(runner, "d", ids, [20] + [1] * 17), want) < 2e-5
    assert err(feed(runner, "p", ids, [2, 3, 2, 9, 2, 7, 5, 2, 5]), want) < 2e-5


# ---------------------------------------------------------------- the engine on the stand-in kernels (CPU)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_cpu(dirs, name):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32), d, cfg["vocab"], 2e-5)


@pytest.mark.parametrize("name", ["mix", "pages"])
def test_mixed_batches_on_cpu(dirs, name):
    d, cfg, page = dirs[name]
    check_mixed(lambda pages: engine(d, page, pages), d, cfg["vocab"], page, 2e-5)


def test_a_batch_does_not_change_its_members(dirs):
    d, cfg, page = dirs["mix"]
    runner = engine(d, page, 64)
    a, b, c = (tokens(cfg["vocab"], n, seed=n) for n in (19, 7, 30))
    alone = [feed(runner, i, ids, [len(ids)]) for i, ids in enumerate((a, b, c))]
    seqs = [runner.cache.admit(k) for k in "abc"]
    first = runner.step([StepEntry(seqs[0], a[:10], range(10)), StepEntry(seqs[1], b, range(7)), StepEntry(seqs[2], c[:1], [0])])
    second = runner.step([StepEntry(seqs[2], c[1:], range(29)), StepEntry(seqs[0], a[10:11], [0])])
    third = runner.step([StepEntry(seqs[0], a[11:], range(8))])
    got_a = torch.cat([first[:10], second[29:30], third])
    got_c = torch.cat([first[17:18], second[:29]])
    assert err(got_a, alone[0]) < 1e-5 and err(first[10:17], alone[1]) < 1e-5 and err(got_c, alone[2]) < 1e-5


def test_a_freed_slot_starts_from_zero(dirs):
    """A request that takes the slot (and pages) another one just gave back must not see what that one left."""
    d, cfg, page = dirs["ones"]
    runner = engine(d, page, 16, max_seqs=1)
    a, b = tokens(cfg["vocab"], 26, seed=1), tokens(cfg["vocab"], 11, seed=2)
    feed(runner, "a", a, [26])
    assert err(feed(runner, "b", b, [4, 1, 1, 5]), plain_logits(d, b)) < 2e-5


def llm_cpu(d, **kw):
    kw.setdefault("kv_cache_tokens", 512)
    return LLM(d, dtype="float32", device="cpu", ops=TorchRefOps(), **kw)


def plain_greedy(d, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain_logits(d, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("chunked", [False, True])
def test_generate_through_the_entry_point_on_cpu(dirs, chunked):
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=40 + n) for n in (5, 13, 22, 9, 3)]
    want = [plain_greedy(d, p, 6) for p in prompts]
    llm = llm_cpu(d, kv_block_size=page, max_num_seqs=3, chunked_prefill=chunked, max_batched_tokens=16 if chunked else 64)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert got == want
    assert llm.cache.free_pages() == llm.cache.num_pages and llm.cache.slots.num_free == 3


def test_preemption_recomputes_state(dirs):
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=60 + n) for n in (14, 15, 13)]
    want = [plain_greedy(d, p, 8) for p in prompts]
    llm = llm_cpu(d, kv_block_size=page, kv_cache_tokens=56, max_num_seqs=3, kv_watermark=0.0)
    assert llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True)) == want
    assert llm.scheduler.preemptions > 0


def test_trace_replay_in_process(dirs, tmp_path, monkeypatch, capsys):
    from mini_inference_b200.cli import trace_run
    d, cfg, page = dirs["pages"]
    a, b = tokens(cfg["vocab"], 9, seed=1), tokens(cfg["vocab"], 6, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:5], "want": [4]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 3]}, {"id": "a", "tokens": a[5:6], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[6:], "want": [2]}], "end": ["a"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    monkeypatch.setattr("mini_inference_b200.engine.factory.make_runner",
                        lambda model, *a_, **k: make_runner(model, *a_, **{**k, "ops": TorchRefOps()}))
    assert trace_run.main(["--model", d, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128", "--device", "cpu",
                           "--page-size", str(page)]) == 0
    assert [line for line in capsys.readouterr().out.split("\n") if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = plain_logits(d, a), plain_logits(d, b)
    g0 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "0.f32"), dtype="<f4").reshape(1, -1))
    g1 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "1.f32"), dtype="<f4").reshape(3, -1))
    g2 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "2.f32"), dtype="<f4").reshape(1, -1))
    assert err(g0, wa[4:5]) < 2e-5 and err(g1, torch.stack([wb[2], wb[5], wa[5]])) < 2e-5 and err(g2, wa[8:9]) < 2e-5


# ---------------------------------------------------------------- inputs made so that a fault shows
def hot_key_case(ops, device, dtype, L, hot, block, page, rows=1, H=4, KV=2, D=24, V=16, sink=True, window=None):
    """L cached keys; the entry feeds the last `rows` positions (rows = 1: a decoded token) and the LAST query is looked at.
    Every key is orthogonal to the query's direction except key `hot`, whose score stands out by 30.  If `hot` is one of the
    keys the query may see, the output is that key's value; if not, every visible score is 0 and, with the sink's extra term,
    the output is the sum of the n visible values / (n + 1)."""
    g = torch.Generator().manual_seed(L * 1000 + hot)
    keys, vals = torch.randn(L, KV, D, generator=g) * 0.3, torch.randn(L, KV, V, generator=g)
    target = torch.randn(D, generator=g)
    target = target / target.norm()
    keys -= (keys @ target)[..., None] * target
    keys[hot] += 6.0 * target
    pages = -(-L // page)
    order = torch.randperm(pages, generator=g) + 1               # pages in a shuffled order (page 0 is the null page)
    kc, vc = torch.zeros(pages + 1, KV, page, D), torch.zeros(pages + 1, KV, page, V)
    for j in range(L):
        kc[order[j // page], :, j % page], vc[order[j // page], :, j % page] = keys[j], vals[j]
    table = torch.zeros(2, pages, dtype=torch.int32)
    table[1] = order.to(torch.int32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)      # noqa: E731
    tiles = [(0, r) for r in range(0, rows, 64)] if rows > 1 else []
    meta = SimpleNamespace(seg_q_start=i32([0, rows]), seg_pos0=i32([L - rows]), seg_kv_len=i32([L]), table_rows=i32([1]),
                           block_table=table.to(device), max_pages=pages, page_size=page, decode_segs=i32([0] if rows == 1 else []),
                           prefill_tiles=i32(tiles).view(-1, 2), tile=64, max_kv_len=L)
    q = torch.randn(rows, H, D, generator=g)
    q[-1] = 5.0 * target
    out = ops.masked_attention(q.reshape(rows, H * D).to(device, dtype), kc.to(device, dtype), vc.to(device, dtype), meta, H, KV, D, V,
                               1.0, block, window, sink).float().cpu()[-1].view(H, V)
    p = L - 1
    lo = 0 if not block else (p // block) * block
    if window:
        lo = max(lo, p - window + 1)
    kvh = torch.arange(H) // (H // KV)
    want = vals[hot][kvh] if hot >= lo else vals[lo:].sum(0)[kvh] / (L - lo + (1 if sink else 0))
    return out, want


# (keys, the hot key, block): far back inside the block; first and last key of the block; the key just outside it; at page
# borders; the first keys of the sequence; a block that has just begun (the query sees itself alone)
HOT = [(300, 0, 512), (300, 7, 512), (257, 256, 64), (257, 255, 64), (256, 192, 64), (256, 191, 64), (129, 128, 16), (129, 127, 16),
       (200, 150, 50), (200, 149, 50), (64, 15, 48), (64, 48, 48), (64, 47, 48), (5, 4, 3), (5, 2, 3), (7, 0, None), (90, 3, None)]


@pytest.mark.parametrize("L,hot,block", HOT)
@pytest.mark.parametrize("rows", [1, 3])
def test_keys_at_block_edges_on_cpu(L, hot, block, rows):
    out, want = hot_key_case(TorchRefOps(), "cpu", torch.float32, L, hot, block, page=16, rows=min(rows, L))
    assert (out - want).abs().max() < 1e-3 * want.abs().max() + 1e-6


def test_the_sink_takes_the_weight_when_no_key_matches():
    """Scores of -30 everywhere: without the sink the output would be an average of the values; with it, next to nothing."""
    out, _ = hot_key_case(TorchRefOps(), "cpu", torch.float32, 40, 39, None, page=8)
    assert out.abs().max() > 0.1
    ops = TorchRefOps()
    g = torch.Generator().manual_seed(1)
    k, v = torch.ones(2, 1, 8, 4), torch.randn(2, 1, 8, 6, generator=g)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32)           # noqa: E731
    meta = SimpleNamespace(seg_q_start=i32([0, 1]), seg_pos0=i32([7]), seg_kv_len=i32([8]), table_rows=i32([0]), block_table=i32([[1]]),
                           max_pages=1, page_size=8, decode_segs=i32([0]), prefill_tiles=i32([]).view(-1, 2), tile=64, max_kv_len=8)
    q = torch.full((1, 4), -7.5)
    assert ops.masked_attention(q, k, v, meta, 1, 1, 4, 6, 1.0, None, None, True).abs().max() < 1e-10
    assert ops.masked_attention(q, k, v, meta, 1, 1, 4, 6, 1.0, None, None, False).abs().max() > 1e-2


def far_write_case(ops, device):
    """A head with decay 0.999 must still carry a write from 400 tokens back (0.999^400 = 0.67), a head with decay 0.5 must
    not; whole, with the reading token decoded alone, and in portions.  The rotation turns write and read by their
    positions: the read-out is the cosine of the angle between them."""
    H, D, V, T = 2, 4, 6, 401
    p = torch.zeros(T, 2 * H * D + H * V)
    p[0, H * D:2 * H * D] = torch.tensor([4.0, 0.0, 0.0, 0.0]).repeat(H)      # token 0 writes key e_0 * 4 ...
    p[0, 2 * H * D:] = 3.0                                                    # ... with value 3 in both heads
    p[T - 1, :H * D] = torch.tensor([2.0, 0.0, 0.0, 0.0]).repeat(H)           # the last token reads with query e_0 * 2
    decay = torch.tensor([0.999, 0.5]).to(device)
    inv_freq = torch.tensor([0.01]).to(device)                                # coordinates 0 and 1 form the one rotated pair
    want0 = 4.0 * 0.5 * 3.0 * 2.0 * 0.999 ** 400 * math.cos(400 * 0.01)
    for cuts in ([T], [T - 1, 1], [200, 150, 50, 1]):
        state = torch.zeros(2, H * D * V, device=device)
        outs, at = [], 0
        for n in cuts:
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)      # noqa: E731
            batch = SimpleNamespace(host={"seg_q_start": [0, n], "seg_slot": [1]}, num_segs=1, seg_q_start=i32([0, n]), seg_slot=i32([1]),
                                    positions=i32(list(range(at, at + n))))
            outs.append(ops.retention_scan(p[at:at + n].to(device), H, D, V, inv_freq, 0.5, decay, state, batch).cpu())
            at += n
        o = torch.cat(outs)[T - 1].view(H, V)
        assert torch.allclose(o[0], torch.full((V,), want0), rtol=2e-4) and o[1].abs().max() < 1e-15


def test_retention_remembers_a_far_token_on_cpu():
    far_write_case(TorchRefOps(), "cpu")


def test_value_blend_takes_the_source_layers_values(tmp_path):
    """lambda = 1 in the blending layer: its own value projection must not matter at all."""
    d = single_dir(tmp_path, "attention_blend")
    from mini_inference_b200.weights.safetensors_io import write_safetensors
    cfg, w = plain.load_model_dir(d)
    w["l1.mix.vmix"] = torch.ones((), dtype=w["l1.mix.vmix"].dtype)
    ids = tokens(cfg["vocab"], 19, seed=2)
    outs = []
    for scale in (1.0, -3.0):
        w2 = dict(w)
        w2["l1.mix.v"] = w["l1.mix.v"] * scale
        write_safetensors(os.path.join(d, "model.safetensors"), [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in w2.items()])
        outs.append(feed(engine(d, 4, 16), "a", ids, [7, 1, 1, 10]))
        _PLAIN.pop(d, None)
        assert err(outs[-1], plain_logits(d, ids)) < 2e-5
    assert err(outs[0], outs[1]) < 1e-6


# ================================================================ on the GPU
gpu = pytest.mark.gpu
TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def cuda_ops():
    from mini_inference_b200.ops import get_ops
    return get_ops("cuda:0")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32, dtype, "cuda:0"), d, cfg["vocab"], TOL[dtype])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "pages", "rows64"])
def test_mixed_batches_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_mixed(lambda pages: engine(d, page, pages, dtype, "cuda:0"), d, cfg["vocab"], page, TOL[dtype])
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone_on_gpu(tmp_path, name, dtype):
    cfg = SINGLE[name]
    d = single_dir(tmp_path, name)
    ids = tokens(cfg["vocab"], 150, seed=1)
    want = plain_logits(d, ids)
    runner = engine(d, 16, 16, dtype, "cuda:0")
    assert_close(feed(runner, "w", ids, [150]), want, TOL[dtype])
    assert_close(feed(runner, "d", ids, [110] + [1] * 40), want, TOL[dtype])
    assert_close(feed(runner, "p", ids, [2, 64, 3, 17, 2, 33, 29]), want, TOL[dtype])


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,hot,block", HOT + [(1500, 31, 2048), (1500, 1023, 1024), (1500, 1024, 1024)])
def test_keys_at_block_edges_on_gpu(L, hot, block, dtype):
    ops = cuda_ops()
    for D, V in ((24, 16), (64, 64), (128, 128)):        # equal rows of 64 or 128 entries: the tensor-core prompt kernel in bfloat16
        for rows in (1, 3, 70):
            for splits in (None, 3):
                ops.force_splits = splits
                try:
                    out, want = hot_key_case(ops, "cuda:0", dtype, L, hot, block, page=16, rows=min(rows, L), D=D, V=V)
                finally:
                    ops.force_splits = None
                assert (out - want).abs().max() < (1e-3 if dtype == torch.float32 else 2e-2) * want.abs().max() + 1e-6


@gpu
def test_retention_remembers_a_far_token_on_gpu():
    far_write_case(cuda_ops(), "cuda:0")


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernels_against_the_stand_ins(dtype):
    """Every new kernel alone at sizes no model above has, against the plain PyTorch statement of the same op."""
    ops, ref, dev = cuda_ops(), TorchRefOps(), "cuda:0"
    g = torch.Generator().manual_seed(0)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype)      # noqa: E731
    f32 = lambda *s: torch.randn(*s, generator=g)                # noqa: E731
    close = lambda a, b, t=tol: (a.float().cpu() - b.float().cpu()).abs().max() <= t * max(1.0, b.float().abs().max().item())  # noqa: E731
    # stream kernels
    ids, table = torch.randint(0, 50, (9,), generator=g, dtype=torch.int32), rnd(50, 77)
    xa, ra = ops.embed_stream(ids.to(dev), table.to(dev), dtype)
    xb, rb = ref.embed_stream(ids, table, dtype)
    assert xa.dtype == torch.float32 and ra.dtype == dtype and close(xa, xb, 0) and close(ra, rb, 0)
    y, w, ls = rnd(9, 77), f32(77), f32(77)
    for scale in (ls, None):
        ra = ops.out_rmsnorm_add(xa, y.to(dev), w.to(dev), None if scale is None else scale.to(dev), 0.3, 1e-5, dtype)
        rb = ref.out_rmsnorm_add(xb, y, w, scale, 0.3, 1e-5, dtype)
        assert close(xa, xb, 2e-6) and close(ra, rb)
    rows, dl = torch.tensor([8, 2], dtype=torch.int32), rnd(9, 77)
    assert close(ops.stream_rmsnorm(xa, None, w.to(dev), 1e-5, rows.to(dev), dtype), ref.stream_rmsnorm(xb, None, w, 1e-5, rows, dtype))
    assert close(ops.stream_rmsnorm(xa, dl.to(dev), w.to(dev), 1e-5, None, dtype), ref.stream_rmsnorm(xb, dl, w, 1e-5, None, dtype))
    assert close(xa, xb, 2e-6)
    if dtype == torch.bfloat16:
        assert close(ops.cast_rows(xa, dtype), xb.to(dtype), 0)
    o, gate = f32(6, 3 * 10), rnd(6, 50)
    assert close(ops.group_rmsnorm_gate(o.to(dev), None, gate.to(dev)[:, 7:37], 1e-5, 3, 10, dtype, act="silu"),
                 ref.group_rmsnorm_gate(o, None, gate[:, 7:37], 1e-5, 3, 10, dtype, act="silu"))
    # q/k unit norms, value blend, cache write: slots out of order over shuffled pages
    H, KV, D, V, page, T = 5, 1, 24, 40, 8, 11
    p, src, lam = rnd(T, (H + KV) * D + KV * V), rnd(T, KV * V + 5), torch.tensor([0.3])
    slots = (torch.randperm(40, generator=g)[:T] + 8).to(torch.int32)
    for source in (None, src[:, 5:]):
        ka, va = torch.zeros(7, KV, page, D, dtype=dtype, device=dev), torch.zeros(7, KV, page, V, dtype=dtype, device=dev)
        kb, vb = ka.cpu(), va.cpu()
        meta = SimpleNamespace(slots=slots, page_size=page)
        qa = ops.unit_qk_cache(p.clone().to(dev), H, KV, D, V, 1e-5, lam.to(dev), None if source is None else source.to(dev),
                               SimpleNamespace(slots=slots.to(dev), page_size=page), ka, va)
        qb = ref.unit_qk_cache(p.clone(), H, KV, D, V, 1e-5, lam, source, meta, kb, vb)
        assert close(qa, qb) and close(ka, kb) and close(va, vb)
    # retention: three entries of unequal length in one launch, states that start non-zero, slots out of order
    lens, slots3, qs, T = [1, 23, 6], [3, 1, 2], [0, 1, 24, 30], 30
    pos = [40] + list(range(5, 28)) + list(range(100, 106))
    batch = SimpleNamespace(host={"seg_q_start": qs, "seg_slot": slots3}, num_segs=3, positions=torch.tensor(pos, dtype=torch.int32))
    dbatch = SimpleNamespace(seg_q_start=torch.tensor(qs, dtype=torch.int32, device=dev), seg_slot=torch.tensor(slots3, dtype=torch.int32, device=dev),
                             positions=batch.positions.to(dev), num_segs=3)
    for H, D, V, half in ((3, 10, 37, 3), (2, 33, 8, 16), (1, 130, 40, 65), (2, 6, 5, 0)):
        p, decay, st = rnd(T, 2 * H * D + H * V + 3), torch.rand(H, generator=g), f32(4, H * D * V)
        inv = torch.rand(half, generator=g) if half else None
        sa, sb = st.clone().to(dev), st.clone()
        oa = ops.retention_scan(p.to(dev), H, D, V, None if inv is None else inv.to(dev), D ** -0.5, decay.to(dev), sa, dbatch)
        assert close(oa, ref.retention_scan(p, H, D, V, inv, D ** -0.5, decay, sb, batch), 1e-4 if dtype == torch.float32 else tol)
        assert close(sa, sb, 1e-4)
    # router and experts
    for T, hid, E, top, groups, F in ((13, 44, 6, 2, (3, 2), 10), (70, 128, 16, 5, (4, 2), 64), (5, 33, 7, 7, None, 9), (40, 64, 8, 1, (8, 1), 64),
                                      (300, 64, 4, 2, None, 192), (1100, 72, 6, 2, (3, 2), 8), (900, 320, 5, 3, None, 576)):
        h, router, corr = rnd(T, hid), rnd(E, hid) * 0.5, f32(E) * 0.2
        ca, wa = ops.route_topk(h.to(dev), router.to(dev), corr.to(dev), top, groups)
        cb, wb = ref.route_topk(h, router, corr, top, groups)
        assert torch.equal(ca.cpu(), cb) and close(wa, wb, 1e-5)
        w_in, w_out, shared = rnd(E, 2 * F, hid) * 0.3, rnd(E, hid, F) * 0.3, rnd(T, hid)
        for sh in (None, shared):
            # bfloat16: the CUDA-core form, the mma.sync form, and (where an expert gets many rows) the tcgen05 form
            for tc, tc5 in (((False, False), (True, False), (True, True)) if dtype == torch.bfloat16 else ((False, False),)):
                keep = (ops.moe_tc, ops.moe_tcgen05)
                ops.moe_tc, ops.moe_tcgen05 = tc and keep[0], tc5 and keep[1]
                try:
                    got = ops.expert_ffn(h.to(dev), ca, wa, w_in.to(dev), w_out.to(dev), 1.3, 1.702, None if sh is None else sh.to(dev))
                finally:
                    ops.moe_tc, ops.moe_tcgen05 = keep
                assert close(got, ref.expert_ffn(h, cb, wb, w_in, w_out, 1.3, 1.702, sh))
        gu = rnd(T, 2 * F) * 3
        assert close(ops.clamped_glu(gu.to(dev), 1.3, 1.702), ref.clamped_glu(gu, 1.3, 1.702))
    ops.check_errors()


@gpu
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_through_the_entry_point_on_gpu(dirs, dtype, graphs):
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=40 + n) for n in (5, 13, 22, 9, 3, 30)]
    llm = LLM(d, dtype=dtype, kv_block_size=page, kv_cache_tokens=1024, max_num_seqs=4, cuda_graphs=graphs)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert llm.cache.free_pages() == llm.cache.num_pages
    if graphs:
        assert llm.graphs.replays > 0
    if dtype == "float32":
        assert got == [plain_greedy(d, p, 12) for p in prompts]
    else:                                                        # judged by logits, not by token prefixes
        for p, out in zip(prompts, got):
            logits = plain_logits(d, p + out)
            for i, tok in enumerate(out):
                row = logits[len(p) + i - 1]
                assert row[tok] >= row.max() - 0.12 * row.abs().max()


@gpu
def test_trace_run_program_on_gpu(dirs, tmp_path):
    d, cfg, page = dirs["pages"]
    a = tokens(cfg["vocab"], 70, seed=5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[64:], "want": [5]}], "end": ["a"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        want = plain_logits(d, a)
        g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
        g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1))
        assert_close(torch.cat([g0, g1]), want[[0, 63, 69]], TOL[dtype])
