"""The Lilenex decoder through the engine's host side, without a GPU: configuration, registry, weight names, the
cache's kept first pages and shared entries, and -- with the plain PyTorch operator set of tests/torch_ops.py in place
of the CUDA kernels -- every way of cutting requests into steps against the whole-sequence plain implementation of
tests/plain_lilenex.py."""
import copy
import json

import pytest
import torch

import plain_lilenex as plain
import traces
from conftest import random_tokens
from torch_ops import TorchOps
from pytriton_llama_b200.cache.manager import CacheManager
from pytriton_llama_b200.config import ConfigError, EngineConfig, LilenexConfig, resolve_architecture
from pytriton_llama_b200.engine.engine import Engine, StepEntry
from pytriton_llama_b200.parts.base import CacheNeed

TOL = 2e-4      # float32 operators against float64


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg=None, seed=5):
        if name not in made:
            folder = tmp_path_factory.mktemp(f"lilenex_{name}")
            plain.write_model(folder, cfg or plain.TINY[name], seed)
            made[name] = folder
        return made[name]
    return get


def _engine(folder, page, pages, max_seq_len=256, slots=4):
    cfg = EngineConfig(dtype="float32", page_size=page, max_gpu_num_blocks=pages, max_seq_len=max_seq_len, max_num_seqs=slots)
    return Engine(folder, cfg, device="cpu", ops=TorchOps())


def _reference(folder, seqs):
    from pytriton_llama_b200.weights import read_folder
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    return {r: plain.forward(cfg, W, s) for r, s in seqs.items()}


def _seqs(lengths, vocab, seed):
    return {f"r{i}": random_tokens(n, vocab, seed * 100 + i) for i, n in enumerate(lengths)}


def _close(got, want, tol=TOL):
    err = (got.double() - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), err


# ---------------------------------------------------------------------------- configuration and names
def test_config_reads_every_key_and_round_trips():
    cfg = LilenexConfig.from_dict(plain.TINY_A)
    assert (cfg.vocab, cfg.width, cfg.streams, cfg.residual_mult, cfg.norm_eps) == (97, 48, 2, 0.7, 1e-5)
    assert [L.type for L in cfg.layers] == ["attention", "gla", "attention", "attention"] and cfg.layers[3].mlp is None
    a = cfg.layers[2].mixer
    assert (a.window, a.keep_first, a.kv_from, a.rot.dims, a.rot.scaling.factor) == (19, 5, 0, 8, 4.0)
    assert cfg.layers[3].mixer.window == 0 and cfg.layers[3].mixer.rot.scaling is None
    assert (cfg.layers[1].mlp.experts, cfg.layers[1].mlp.top, cfg.layers[1].mlp.shared_ff, cfg.layers[2].mlp.shared_ff) == (5, 2, 16, 0)
    assert LilenexConfig.from_dict(cfg.to_dict()) == cfg
    assert LilenexConfig.from_dict(plain.TINY_B).streams == 0
    assert resolve_architecture(plain.TINY_A).name == "Lilenex"


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0].update(type="conv"), lambda c: c["layers"][0]["mixer"].update(heads=5),
    lambda c: c["layers"][0]["mlp"].update(kind="sparse"), lambda c: c["norm"].update(eps=0), lambda c: c.update(layers=[]),
    lambda c: c["layers"][2]["mixer"].update(kv_from=1), lambda c: c["layers"][2]["mixer"].update(kv_from=3),
    lambda c: c["layers"][2]["mixer"].update(vdim=8), lambda c: c["layers"][1]["mlp"]["router"].update(top=9),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), lambda c: c["layers"][1]["mixer"].update(tau=0),
])
def test_config_names_what_is_wrong(change):
    bad = copy.deepcopy(plain.TINY_A)
    change(bad)
    with pytest.raises(ConfigError):
        LilenexConfig.from_dict(bad)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_the_model_expects_the_checkpoint_names_and_shapes(name):
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY[name])
    model = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY[name])), Runtime(torch.device("cpu"), torch.float32, None))
    want = plain.tensor_shapes(plain.TINY[name])
    got = {k: tuple(v.shape) for k, v in model.expected_tensors().items()}
    assert set(got) == set(want)
    for k, shape in got.items():        # (a negative size is one that only the checkpoint fixes)
        assert len(shape) == len(want[k]) and all(a < 0 or a == b for a, b in zip(shape, want[k])), k


def test_a_layer_that_reads_anothers_keys_shares_its_cache_entry_with_the_wider_need():
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY_A)
    spec = arch.spec_from_config(arch.config_from_dict(plain.TINY_A))
    assert [(e.layer, e.cache, e.write) for e in spec.run_order] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    needs = DecoderModel(spec, Runtime(torch.device("cpu"), torch.float32, None)).cache_entries()
    assert (needs[0].kind, needs[0].window, needs[0].keep_first, needs[0].v_dim) == ("window", 19, 5, 24)
    assert needs[1].kind == "none" and needs[1].states == (("S", (3, 8, 12)),)
    assert needs[3].kind == "full"


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from pytriton_llama_b200.weights import read_folder, write_random_model
    folder = write_random_model(tmp_path / "m", plain.TINY_A, seed=3, dtype=torch.float32, std=0.2)
    cfg = json.loads((folder / "config.json").read_text())
    W = read_folder(folder)
    toks = random_tokens(30, 97, 2)
    eng = _engine(folder, 8, 24)
    got = traces.replay(eng, traces.portions({"x": toks}))["x"]
    _close(got, plain.forward(cfg, W, toks))


# ---------------------------------------------------------------------------- the cache: kept first pages
def test_pages_of_kept_first_positions_stay_and_passed_ones_come_back():
    need = CacheNeed(kind="window", kv_heads=1, head_dim=8, window=10, keep_first=5)
    cm = CacheManager({0: need}, page_size=4, num_pages=12, max_requests=2, max_seq_len=200, device="cpu", dtype=torch.float32)
    cm.admit("a")
    cm.append("a", 30)
    cm.append("a", 1)          # the query at position 30 sees 21..30 and 0..4: blocks 0, 1 stay, 2..4 go, 5.. stay
    table = cm.block_table("a", 0)
    assert [p >= 0 for p in table] == [True, True, False, False, False, True, True, True]
    cm.check_invariants()
    assert cm.free_pages(0) == 12 - 5
    for _ in range(40):
        cm.append("a", 1)
        cm.check_invariants()
    assert cm.free_pages(0) >= 12 - 6 and cm.block_table("a", 0)[0] >= 0 and cm.block_table("a", 0)[1] >= 0
    cm.release("a")
    assert cm.free_pages(0) == 12


# ---------------------------------------------------------------------------- every cut equals the whole sequence
@pytest.mark.parametrize("name,page", [("A", 4), ("A", 16), ("B", 8), ("C", 4)])
def test_every_cut_of_the_requests_matches_the_plain_implementation(folders, name, page):
    folder = folders(name)
    vocab = plain.TINY[name]["vocab"]
    seqs = _seqs([41, 1, 23, 58, 9], vocab, 21)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.prefill_then_decode(seqs, 12), traces.portions(seqs), traces.mixed(seqs)):
        eng = _engine(folder, page, max(40, traces.max_live_tokens(steps, page) // page + 8))
        got = traces.replay(eng, steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


def test_six_requests_through_four_slots_and_few_pages_reuse_what_was_freed(folders):
    folder = folders("A")
    seqs = _seqs([30, 17, 44, 5, 26, 38], 97, 4)
    want = _reference(folder, seqs)
    steps = traces.mixed(seqs, live=3)
    pages = traces.max_live_tokens(steps, 4) // 4 + 2
    eng = _engine(folder, 4, pages, slots=3)
    got = traces.replay(eng, steps)
    for rid in seqs:
        _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])
    assert eng.cache.free_slots() == 3 and all(eng.cache.free_pages(g) == pages for g, grp in enumerate(eng.cache.groups) if grp.paged)


def test_an_unequal_batch_equals_each_request_alone(folders):
    folder = folders("C")
    seqs = _seqs([33, 2, 14], 50, 8)
    eng = _engine(folder, 8, 40)
    together = eng.step([StepEntry(r, s, list(range(len(s)))) for r, s in seqs.items()]).logits
    eng.finish_all()
    at = 0
    for r, s in seqs.items():
        alone = eng.step([StepEntry(r, s, list(range(len(s))))]).logits
        eng.finish(r)
        assert torch.allclose(together[at:at + len(s)], alone, atol=1e-5, rtol=1e-5)
        at += len(s)


def test_long_decoding_token_by_token_past_windows_and_kept_positions(folders):
    folder = folders("A")
    toks = random_tokens(150, 97, 13)
    want = _reference(folder, {"x": toks})["x"]
    eng = _engine(folder, 4, 60)
    rows = [eng.step([StepEntry("x", [t], [0])]).logits[0] for t in toks]
    _close(torch.stack(rows), want)


# ---------------------------------------------------------------------------- each mechanism alone
def _one_layer(mixer_kind, mixer, mlp, streams=0, mult=1.0, width=32):
    return plain.config(41, width, [plain.layer(mixer_kind, mixer, mlp)], streams=streams, mult=mult)


ALONE = {
    "window_keep": _one_layer("attention", plain.attention(2, 1, 8, 8, 0.4, size=6, keep_first=2), None),
    "rotation_part": _one_layer("attention", plain.attention(2, 2, 12, 8, 0.4, rot=plain.rotation(4, 20.0)), None),
    "rotation_yarn": _one_layer("attention", plain.attention(2, 2, 16, 8, 0.4, rot=plain.rotation(16, 100.0, (8.0, 24, 6.0, 0.5))), None),
    "gla": _one_layer("gla", plain.gla(2, 12, 20, 3.0), None),
    "dense": _one_layer("gla", plain.gla(1, 8, 8, 8.0), plain.dense(24)),
    "moe_top1": _one_layer("gla", plain.gla(1, 8, 8, 8.0), plain.moe(12, 7, 1)),
    "moe_top3_shared": _one_layer("gla", plain.gla(1, 8, 8, 8.0), plain.moe(12, 4, 3, shared=20)),
    "streams1": _one_layer("gla", plain.gla(1, 8, 8, 8.0), plain.dense(16), streams=1, mult=0.5),
    "streams5": _one_layer("attention", plain.attention(2, 1, 8, 8, 0.4), plain.dense(16), streams=5, mult=1.5),
}


@pytest.mark.parametrize("name", sorted(ALONE))
def test_each_mechanism_alone_in_a_one_layer_model(folders, name):
    folder = folders("alone_" + name, ALONE[name], seed=3)
    seqs = _seqs([27, 12], 41, 6)
    want = _reference(folder, seqs)
    for steps in (traces.whole(seqs), traces.portions(seqs, sizes=(3, 2, 9, 2))):
        got = traces.replay(_engine(folder, 4, 30), steps)
        for rid in seqs:
            _close(got[rid], want[rid][traces.wanted_positions(steps, rid)])


def test_the_plain_rotation_scales_frequencies_between_the_two_turn_counts():
    f, amp = plain.rotary_frequencies(plain.rotation(16, 100.0, (8.0, 24, 6.0, 0.5)))
    base = 100.0 ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
    assert amp == pytest.approx(0.1 * 2.0794415416798357 + 1.0)
    assert f[0] == base[0] and f[-1] == pytest.approx(float(base[-1]) / 8.0)        # fast pairs untouched, slow ones divided
    assert all(base[i] / 8.0 - 1e-15 <= f[i] <= base[i] + 1e-15 for i in range(8))
    from pytriton_llama_b200.parts.window_attention import yarn_pair_frequencies
    g, amp2 = yarn_pair_frequencies(16, 100.0, {"factor": 8.0, "original": 24, "fast": 6.0, "slow": 0.5})
    assert torch.allclose(f, g, rtol=1e-14, atol=0) and amp == amp2


# ---------------------------------------------------------------------------- generation through the public entry point
def test_greedy_generation_through_the_scheduler_matches_the_plain_argmax(folders):
    from pytriton_llama_b200 import LLM, SamplingParams
    folder = folders("B")
    from pytriton_llama_b200.weights import read_folder
    W = read_folder(folder)
    prompts = list(_seqs([9, 21, 3], 70, 17).values())
    llm = LLM(folder, EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=40, max_seq_len=64, max_num_seqs=2,
                                   max_batched_tokens=8, compiled_model=False), device="cpu", ops=TorchOps())
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_gen_len=7))
    for p, out in zip(prompts, got):
        logits = plain.forward(plain.TINY_B, W, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 1e-4, (i, tok, int(row.argmax()))
