"""Naditar in the engine against the plain implementation (tests/plain/naditar_plain.py).

Without a GPU the engine runs on the stand-in kernel namespace (tests/ref_ops.py), which
exercises configuration, weights, spec, parts, cache and state manager, batch builder,
scheduler and entry point.  With a GPU (-m gpu) the same checks run on the CUDA kernels in
float32 and bfloat16, plus each kernel alone against the plain function of its mechanism."""
import json
import os
import random
import subprocess
import sys

import pytest
import torch

from mini_inference_b200 import LLM, SamplingParams
from mini_inference_b200.config import ConfigError, NaditarConfig, load_config, resolve
from mini_inference_b200.engine.batch import StepEntry
from mini_inference_b200.engine.factory import load_model, make_runner
from mini_inference_b200.models.naditar import execution_order
from mini_inference_b200.weights import write_random_model
from tests.plain import naditar_plain as plain
from tests.ref_ops import TorchRefOps

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def delta(heads, kv, dim, vdim, conv, ff=None, rank=5):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
                                               "decay_rank": rank, "gate_rank": rank + 2},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def light(heads, dim, vdim, decay, ff=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def latent(heads, dim, rot_dim, vdim, rank, base=10000.0, dims=None, ff=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank,
                      "scale": (dim + rot_dim) ** -0.5, "rot": {"base": base, "dims": dims or rot_dim}},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, loop=None, eps=1e-5):
    c = {"architecture": "Naditar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# Small configurations that differ from one another in every size; none of them makes two sizes equal by accident.
CONFIGS = {
    # every mixer once, a looped span in the middle, a layer without feed-forward, key heads shared by value heads
    "mix": (config(48, 131, [light(3, 8, 24, [0.5, 0.9, 0.99], ff=72), delta(4, 2, 8, 12, 3, ff=40),
                             latent(3, 8, 6, 10, 20, dims=4), delta(2, 2, 16, 40, 2)], loop=(1, 3, 2)), 4),
    # the loop starts at the first layer and covers everything; a convolution of one tap; an odd value size
    "loop_all": (config(40, 97, [delta(2, 1, 12, 9, 1, ff=56), light(2, 12, 7, [0.8, 0.97])], loop=(0, 2, 3), eps=1e-6), 8),
    # no loop at all; two latent layers of different sizes (two cache groups); a larger rotary base
    "latents": (config(64, 150, [latent(4, 16, 8, 12, 24, base=1e6, ff=96), latent(2, 8, 16, 20, 48, ff=80),
                                 light(4, 16, 32, [0.6, 0.9, 0.97, 0.999], ff=64)]), 16),
    # a span that runs once (times = 1) after a layer outside it; four taps
    "once": (config(56, 211, [delta(3, 3, 8, 16, 4, ff=64), latent(2, 12, 4, 8, 16, ff=48), light(2, 8, 8, [0.9, 0.95])],
                    loop=(1, 3, 1)), 4),
}
STD = 0.18          # large enough for every mixer to move the stream by about as much as the stream itself


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (name, (cfg, page)) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("naditar_" + name))
        write_random_model(cfg, d, seed=10 + i, std=STD, norm_init="uniform")
        out[name] = (d, cfg, page)
    return out


def tokens(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_PLAIN = {}


def plain_logits(d, ids):
    if d not in _PLAIN:
        _PLAIN[d] = plain.load_dir(d, torch.float64)
    cfg, w = _PLAIN[d]
    return plain.forward(cfg, w, ids).float()


def err(got, want):
    return ((got - want).abs().max() / want.abs().max()).item()


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
    one by one (long decoding: every state and cache row is written one token at a time)."""
    ids = tokens(vocab, n, seed=3)
    want = plain_logits(d, ids)
    free = runner.cache.free_pages()
    assert err(feed(runner, "w", ids, [n]), want) < tol
    assert err(feed(runner, "d", ids, [n - 24] + [1] * 24), want) < tol
    assert err(feed(runner, "p", ids, portions(n, random.Random(1))), want) < tol
    assert err(feed(runner, "2", ids[:20], [2] * 10), want[:20]) < tol
    assert err(feed(runner, "1", ids, [1] * n), want) < tol
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
    slot_uses = {}
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
        assert err(torch.cat(got[k]), want[k]) < tol, k
    assert runner.cache.free_pages() == pages
    assert len(slot_uses) <= 4 and max(slot_uses.values()) >= 2, "no state slot was used again"


# ---------------------------------------------------------------- configuration, registry, order of layers
def test_config_reads_every_key_and_refuses_what_is_missing():
    raw = CONFIGS["mix"][0]
    assert resolve(raw).name == "Naditar" and resolve({"architectures": ["Naditar"]}).name == "Naditar"
    cfg = NaditarConfig.from_dict(raw)
    assert NaditarConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.loop == (1, 3, 2) and cfg.layers[3].ff is None and cfg.layers[2].mixer_dict()["rot"] == {"base": 10000.0, "dims": 4}
    for path, msg in ((("norm",), "norm"), (("layers", 0, "mixer", "decay"), "decay"), (("layers", 1, "mixer", "conv"), "conv"),
                      (("layers", 2, "mixer", "rot"), "rot"), (("vocab",), "vocab")):
        broken = json.loads(json.dumps(raw))
        node = broken
        for p in path[:-1]:
            node = node[p]
        del node[path[-1]]
        with pytest.raises(ConfigError, match=msg):
            NaditarConfig.from_dict(broken)
    bad = json.loads(json.dumps(raw))
    bad["layers"][0]["type"] = "window_attention"
    with pytest.raises(ConfigError, match="window_attention"):
        NaditarConfig.from_dict(bad)
    bad = json.loads(json.dumps(raw))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        NaditarConfig.from_dict(bad)


def test_execution_order_and_separate_caches(dirs):
    order = execution_order(5, (1, 3, 3))
    assert [(s.layer, s.add_row) for s in order] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None), (4, None)]
    assert [(s.layer, s.add_row) for s in execution_order(2, None)] == [(0, None), (1, None)]
    assert [(s.layer, s.add_row) for s in execution_order(2, (0, 2, 2))] == [(0, 0), (1, None), (0, 1), (1, None)]
    d, cfg, page = dirs["mix"]
    _, spec = load_config(d)
    assert spec.residual == "float32" and spec.pass_vectors_rows == 2
    runner = engine(d, page, 8)
    caches = runner.cache.layer_caches
    assert len(caches) == 6                                    # 1 + 2 x 2 + 1 layer runs
    # the two passes of the looped delta layer hold two states; those of the looped latent layer two planes of one group
    assert caches[1].state.data_ptr() != caches[3].state.data_ptr()
    assert caches[2].group == caches[4].group and caches[2].k.data_ptr() != caches[4].k.data_ptr() and caches[2].v is None


# ---------------------------------------------------------------- each mechanism alone (one layer, no feed-forward)
SINGLE = {
    "lightning": config(32, 61, [light(3, 8, 10, [0.3, 0.9, 0.999])]),
    "lightning_ff": config(32, 61, [light(2, 4, 36, [0.7, 0.95], ff=44)]),
    "channel_delta": config(36, 67, [delta(4, 2, 8, 6, 3)]),
    "channel_delta_taps4": config(36, 67, [delta(2, 2, 20, 33, 4)]),
    "latent": config(40, 71, [latent(3, 8, 6, 10, 12)]),
    "latent_part_rotated": config(40, 71, [latent(2, 4, 12, 6, 20, dims=8, base=100.0)]),
    # cached rows of 64 entries: in bfloat16 on the GPU prompt portions take the tensor-core kernel with split softmax weights
    "latent_rows64": config(40, 71, [latent(3, 8, 16, 10, 48)]),
    # sizes that put every view of a fused product on an odd offset and every row on an odd length
    "lightning_odd": config(27, 53, [light(3, 5, 7, [0.4, 0.8, 0.95])]),
    "channel_delta_odd": config(27, 53, [delta(3, 1, 9, 6, 3, rank=3)]),
    "latent_odd": config(27, 53, [latent(3, 5, 4, 3, 7, dims=2)]),
}


@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name):
    cfg = SINGLE[name]
    d = write_random_model(cfg, str(tmp_path), seed=3, std=0.3, norm_init="uniform")
    ids = tokens(cfg["vocab"], 37, seed=1)
    want = plain_logits(d, ids)
    # the mixer matters: without it the logits are those of the embedding alone
    c0, w = plain.load_dir(d, torch.float64)
    eps = c0["norm"]["eps"]
    bare = (plain.scalar_norm(plain.scalar_norm(w["embed"][torch.tensor(ids)], w["embed.norm"], eps), w["final.norm"], eps) @ w["head"].T).float()
    assert err(bare, want) > 0.05
    runner = engine(d, 4, 16)
    assert err(feed(runner, "w", ids, [37]), want) < 2e-5
    assert err(feed(runner, "d", ids, [20] + [1] * 17), want) < 2e-5
    assert err(feed(runner, "p", ids, [2, 3, 2, 9, 2, 7, 5, 2, 5]), want) < 2e-5


def test_plain_mechanisms_by_hand():
    """The plain functions themselves on inputs whose answer is known."""
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.rms(x, 0.0), x / (12.5 ** 0.5))
    z = torch.tensor([[1.0, -2.0]], dtype=torch.float64)
    got = plain.polynorm(z, [1.0, 10.0, 100.0, 0.5], 0.0)
    want = z / (2.5 ** 0.5) + 10 * z ** 2 / (8.5 ** 0.5) + 100 * z ** 3 / (32.5 ** 0.5) + 0.5
    assert torch.allclose(got, want)
    seq = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    conv = plain.causal_conv(seq, torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64))
    assert conv[:, 0].tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]              # the last tap is the current token's
    r = plain.rotate_interleaved(torch.tensor([[1.0, 0.0, 5.0, 7.0]], dtype=torch.float64), torch.tensor([1]), 2, 10.0)
    assert torch.allclose(r, torch.tensor([[torch.cos(torch.tensor(1.0)).item(), torch.sin(torch.tensor(1.0)).item(), 5.0, 7.0]], dtype=torch.float64))


# ---------------------------------------------------------------- the engine on the stand-in kernels (CPU)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_cpu(dirs, name):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32), d, cfg["vocab"], 2e-5)


@pytest.mark.parametrize("name", ["mix", "latents"])
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
    d, cfg, page = dirs["loop_all"]
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
    """A pool too small for all requests at once: the newest is evicted, its slot zeroed again and its tokens recomputed."""
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=60 + n) for n in (14, 15, 13)]
    want = [plain_greedy(d, p, 8) for p in prompts]
    llm = llm_cpu(d, kv_block_size=page, kv_cache_tokens=56, max_num_seqs=3, kv_watermark=0.0)
    assert llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True)) == want
    assert llm.scheduler.preemptions > 0


def test_trace_replay_in_process(dirs, tmp_path, monkeypatch, capsys):
    import io
    from mini_inference_b200.cli import trace_run
    d, cfg, page = dirs["once"]
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
    import numpy as np
    wa, wb = plain_logits(d, a), plain_logits(d, b)
    g0 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "0.f32"), dtype="<f4").reshape(1, -1))
    g1 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "1.f32"), dtype="<f4").reshape(3, -1))
    g2 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "2.f32"), dtype="<f4").reshape(1, -1))
    assert err(g0, wa[4:5]) < 2e-5 and err(g1, torch.stack([wb[2], wb[5], wa[5]])) < 2e-5 and err(g2, wa[8:9]) < 2e-5


# ---------------------------------------------------------------- inputs made so that a fault shows
def far_key_case(ops, device, dtype, L, far, page, H=3, C=24, R=8):
    """Latent attention over L cached rows of which row `far` alone matches the query of every head: its score stands
    out by ~30, so the output must be that row's first C entries; every other row pulls the output elsewhere."""
    from types import SimpleNamespace
    g = torch.Generator().manual_seed(L * 1000 + far)
    rows = torch.randn(L, C + R, generator=g) * 0.3
    target = torch.randn(C + R, generator=g)
    target = target / target.norm()
    rows -= (rows @ target)[:, None] * target[None, :]           # every row orthogonal to the target direction ...
    rows[far] += 6.0 * target                                    # ... except the far one
    q = (5.0 * target).repeat(H, 1)[None]                        # [1, H, C + R]: score 30 at the far row, ~0 elsewhere
    pages = -(-L // page)
    order = torch.randperm(pages, generator=g) + 1               # pages in a shuffled order (page 0 is the null page)
    cache = torch.zeros(pages + 1, 1, page, C + R)
    for j in range(L):
        cache[order[j // page], 0, j % page] = rows[j]
    table = torch.zeros(2, pages, dtype=torch.int32)
    table[1, :] = order.to(torch.int32)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)      # noqa: E731
    meta = SimpleNamespace(seg_q_start=i32([0, 1]), seg_pos0=i32([L - 1]), seg_kv_len=i32([L]), table_rows=i32([1]),
                           block_table=table.to(device), max_pages=pages, page_size=page, decode_segs=i32([0]),
                           prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device=device), tile=64, max_kv_len=L)
    out = ops.latent_attention(q.to(device, dtype), cache.to(device, dtype), meta, H, C, R, 1.0).float().cpu()
    return out, rows[far, :C]


@pytest.mark.parametrize("L,far", [(300, 0), (300, 7), (257, 255), (256, 16), (129, 128), (64, 15), (5, 4)])
def test_a_far_key_among_hundreds_on_cpu(L, far):
    out, want = far_key_case(TorchRefOps(), "cpu", torch.float32, L, far, page=16)
    assert (out - want).abs().max() < 1e-3 * want.abs().max() + 1e-6


def far_write_case(ops, device):
    """A head with decay 0.999 must still carry a write from 400 tokens back (0.999^400 = 0.67), a head with decay 0.5 must
    not; whole, with the reading token decoded alone, and in portions."""
    from types import SimpleNamespace
    H, D, V, T = 2, 4, 6, 401
    p = torch.full((T, 2 * H * D + H * V), -30.0)                # silu(-30) ~ -3e-12: tokens that write and read next to nothing
    p[0, H * D:2 * H * D] = 4.0                                  # token 0 writes key (4, 4, 4, 4) ...
    p[0, 2 * H * D:] = 3.0                                       # ... with value 3 in both heads
    p[T - 1, :H * D] = 2.0                                       # the last token reads with query 2
    decay = torch.tensor([0.999, 0.5]).to(device)
    silu = torch.nn.functional.silu
    want0 = D * silu(torch.tensor(4.0)) * silu(torch.tensor(3.0)) * silu(torch.tensor(2.0)) * 0.999 ** 400
    for cuts in ([T], [T - 1, 1], [200, 150, 50, 1]):
        state = torch.zeros(2, H * D * V, device=device)
        outs, at = [], 0
        for n in cuts:
            i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)      # noqa: E731
            batch = SimpleNamespace(host={"seg_q_start": [0, n], "seg_slot": [1]}, num_segs=1, seg_q_start=i32([0, n]), seg_slot=i32([1]))
            outs.append(ops.lightning_scan(p[at:at + n].to(device), H, D, V, decay, state, batch).cpu())
            at += n
        o = torch.cat(outs)[T - 1].view(H, V)
        assert torch.allclose(o[0], want0.expand(V), rtol=1e-4) and o[1].abs().max() < 1e-15


def test_lightning_remembers_a_far_token_on_cpu():
    far_write_case(TorchRefOps(), "cpu")


# ================================================================ on the GPU
gpu = pytest.mark.gpu


def cuda_ops():
    from mini_inference_b200.ops import get_ops
    return get_ops("cuda:0")


TOL = {"float32": 1e-4, "bfloat16": 6e-2}


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32, dtype, "cuda:0"), d, cfg["vocab"], TOL[dtype])


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "latents", "loop_all"])
def test_mixed_batches_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_mixed(lambda pages: engine(d, page, pages, dtype, "cuda:0"), d, cfg["vocab"], page, TOL[dtype])
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone_on_gpu(tmp_path, name, dtype):
    cfg = SINGLE[name]
    d = write_random_model(cfg, str(tmp_path), seed=3, std=0.3, norm_init="uniform")
    ids = tokens(cfg["vocab"], 150, seed=1)
    want = plain_logits(d, ids)
    runner = engine(d, 16, 16, dtype, "cuda:0")
    assert err(feed(runner, "w", ids, [150]), want) < TOL[dtype]
    assert err(feed(runner, "d", ids, [110] + [1] * 40), want) < TOL[dtype]
    assert err(feed(runner, "p", ids, [2, 64, 3, 17, 2, 33, 29]), want) < TOL[dtype]


@gpu
def test_kernels_against_the_stand_ins():
    """Every new kernel alone, float32, at sizes no model above has, against the plain PyTorch statement of the same op."""
    from types import SimpleNamespace
    ops, ref, dev = cuda_ops(), TorchRefOps(), "cuda:0"
    g = torch.Generator().manual_seed(0)
    rnd = lambda *s: torch.randn(*s, generator=g)                # noqa: E731
    close = lambda a, b, tol=2e-5: (a.float().cpu() - b.float().cpu()).abs().max() <= tol * max(1.0, b.abs().max().item())  # noqa: E731
    # stream norms
    ids, table, gn = torch.randint(0, 50, (9,), generator=g, dtype=torch.int32), rnd(50, 77), torch.tensor([1.7])
    assert close(ops.embed_scaled_norm(ids.to(dev), table.to(dev), gn.to(dev), 1e-5, torch.float32), ref.embed_scaled_norm(ids, table, gn, 1e-5, torch.float32))
    x, dl, pre, rows = rnd(9, 77), rnd(9, 77), rnd(77), torch.tensor([8, 2], dtype=torch.int32)
    xa, xb = x.clone().to(dev), x.clone()
    assert close(ops.add_scaled_rmsnorm(xa, dl.to(dev), gn.to(dev), 1e-5, None, pre.to(dev), torch.float32), ref.add_scaled_rmsnorm(xb, dl, gn, 1e-5, None, pre, torch.float32))
    assert close(xa, xb)
    assert close(ops.add_scaled_rmsnorm(xa, dl.to(dev), gn.to(dev), 1e-5, rows.to(dev), None, torch.float32), ref.add_scaled_rmsnorm(xb, dl, gn, 1e-5, rows, None, torch.float32))
    assert close(xa, xb)                                         # with rows the stream is left as it is
    z, coef = rnd(5, 301), torch.tensor([0.7, -0.3, 0.2, 0.1])
    assert close(ops.polynorm(z.to(dev), coef.to(dev), 1e-6), ref.polynorm(z, coef, 1e-6))
    o, w, gate = rnd(6, 3 * 10), rnd(10), rnd(6, 50)
    assert close(ops.group_rmsnorm_gate(o.to(dev), w.to(dev), gate.to(dev)[:, 7:37], 1e-5, 3, 10, torch.float32), ref.group_rmsnorm_gate(o, w, gate[:, 7:37], 1e-5, 3, 10, torch.float32))
    oh, hg = rnd(3, 6, 11), rnd(6, 9)
    assert close(ops.head_gate(oh.to(dev), hg.to(dev)[:, 2:5], torch.float32), ref.head_gate(oh, hg[:, 2:5], torch.float32))
    # recurrences: three entries of unequal length in one launch, states that start non-zero, slots out of order
    lens, slots = [1, 23, 6], [3, 1, 2]
    qs = [0, 1, 24, 30]
    T = 30
    batch = SimpleNamespace(host={"seg_q_start": qs, "seg_slot": slots}, num_segs=3)
    dbatch = SimpleNamespace(seg_q_start=torch.tensor(qs, dtype=torch.int32, device=dev), seg_slot=torch.tensor(slots, dtype=torch.int32, device=dev),
                             token_seg=torch.tensor([0] + [1] * 23 + [2] * 6, dtype=torch.int32, device=dev), num_segs=3)
    for H, D, V in ((3, 10, 37), (2, 33, 8), (1, 130, 40)):
        p, decay, st = rnd(T, 2 * H * D + H * V + 3), torch.rand(H, generator=g), rnd(4, H * D * V)
        sa, sb = st.clone().to(dev), st.clone()
        assert close(ops.lightning_scan(p.to(dev), H, D, V, decay.to(dev), sa, dbatch), ref.lightning_scan(p, H, D, V, decay, sb, batch), 1e-4)
        assert close(sa, sb, 1e-4)
    for H, KV, D, V, taps in ((4, 2, 10, 37, 3), (2, 2, 33, 8, 4), (3, 1, 130, 40, 1), (2, 1, 6, 5, 26)):
        C = 2 * KV * D + H * V
        p, a = rnd(T, C + H + 9), rnd(T, H * D)
        conv, A_log, dtb = rnd(C, taps), rnd(H) * 0.3, rnd(H * D)
        st = rnd(4, H * D * V + (taps - 1) * C) * 0.5
        sa, sb = st.clone().to(dev), st.clone()
        pa = ops.delta_prepare(p.to(dev), a.to(dev), conv.to(dev), A_log.to(dev), dtb.to(dev), H, KV, D, V, taps, 1e-6, sa, dbatch)
        pb = ref.delta_prepare(p, a, conv, A_log, dtb, H, KV, D, V, taps, 1e-6, sb, batch)
        n = C + H * D + H                                       # behind these the rows are padding
        assert close(pa[:, :n], pb[:, :n]) and close(sa, sb)                   # the convolutions' last inputs moved into the slots
        assert close(ops.delta_scan(pa, H, KV, D, V, sa, dbatch), ref.delta_scan(pb, H, KV, D, V, sb, batch), 1e-4)
        assert close(sa, sb, 1e-4)
    ops.check_errors()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,far", [(300, 0), (300, 7), (257, 255), (256, 16), (129, 128), (64, 15), (5, 4), (1500, 31), (1500, 1023)])
def test_a_far_key_among_hundreds_on_gpu(L, far, dtype):
    ops = cuda_ops()
    for C, R in ((24, 8), (48, 16), (96, 32)):           # rows of 64 and 128 entries reach the tensor-core decode kernel in bfloat16
        for splits in (None, 3):
            ops.force_splits = splits
            try:
                out, want = far_key_case(ops, "cuda:0", dtype, L, far, page=16, C=C, R=R)
            finally:
                ops.force_splits = None
            assert (out - want).abs().max() < (1e-3 if dtype == torch.float32 else 2e-2) * want.abs().max() + 1e-6


@gpu
def test_split_weight_prompt_attention_against_the_float32_kernel():
    """Latent rows of 64 and 128 entries, bfloat16: prompt portions (on the mma kernel with every softmax weight as two bfloat16
    numbers) beside decoded tokens (float32 kernel) in one step, against the float32 kernels alone on the same inputs."""
    from types import SimpleNamespace
    ops = cuda_ops()
    g = torch.Generator().manual_seed(5)
    for C, R, H in ((48, 16, 3), (96, 32, 5)):
        lens, pos0 = [70, 1, 130, 1], [10, 199, 0, 64]
        page, pages_per = 16, 14
        T = sum(lens)
        cache = (torch.randn(4 * pages_per + 1, 1, page, C + R, generator=g) * 0.5).to("cuda:0", torch.bfloat16)
        table = torch.zeros(5, pages_per, dtype=torch.int32)
        for i in range(4):
            table[i + 1] = torch.randperm(pages_per, generator=g).to(torch.int32) + 1 + i * pages_per
        qs = [0, 70, 71, 201, 202]
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda:0")      # noqa: E731
        tiles = [(i, r) for i, n in enumerate(lens) if n > 1 for r in range(0, n, 64)]
        meta = SimpleNamespace(seg_q_start=i32(qs), seg_pos0=i32(pos0), seg_kv_len=i32([p + n for p, n in zip(pos0, lens)]), table_rows=i32([1, 2, 3, 4]),
                               block_table=table.to("cuda:0"), max_pages=pages_per, page_size=page, decode_segs=i32([1, 3]),
                               prefill_tiles=i32(tiles).view(-1, 2), tile=64, max_kv_len=200)
        q = torch.randn(T, H, C + R, generator=g).to("cuda:0", torch.bfloat16)
        got = ops.latent_attention(q, cache, meta, H, C, R, 0.2).float()
        ops.fast_attention = False
        try:
            want = ops.latent_attention(q, cache, meta, H, C, R, 0.2).float()
        finally:
            ops.fast_attention = True
        assert got.shape == want.shape == (H, T, C)
        assert (got - want).abs().max() <= 2e-2 * want.abs().max()
    ops.check_errors()


@gpu
def test_lightning_remembers_a_far_token_on_gpu():
    far_write_case(cuda_ops(), "cuda:0")


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
    import numpy as np
    d, cfg, page = dirs["latents"]
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
        assert err(g0, want[[0, 63]]) < TOL[dtype] and err(g1, want[69:70]) < TOL[dtype]
