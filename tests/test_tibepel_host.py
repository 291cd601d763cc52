"""The Tibepel decoder through the engine's host side, without a GPU: configuration, registry, weight names, the
cache's named states and block-wise pages, and -- with the plain PyTorch operator set of tests/torch_ops.py in
place of the CUDA kernels -- every way of cutting requests into steps against the whole-sequence plain
implementation of tests/plain_tibepel.py."""
import copy
import json

import pytest
import torch

import plain_tibepel as plain
import traces
from conftest import random_tokens
from torch_ops import TorchOps
from pytriton_llama_b200.cache.manager import CacheManager
from pytriton_llama_b200.config import ConfigError, EngineConfig, TibepelConfig, resolve_architecture
from pytriton_llama_b200.engine.engine import Engine, StepEntry
from pytriton_llama_b200.parts.base import CacheNeed

TOL = 2e-4      # float32 operators against float64, logits capped at 12 to 20


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name, cfg=None, seed=11):
        if name not in made:
            folder = tmp_path_factory.mktemp(f"tibepel_{name}")
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


# ---------------------------------------------------------------------------- configuration and names
def test_config_reads_every_key_and_round_trips():
    cfg = TibepelConfig.from_dict(plain.TINY_Q)
    assert (cfg.vocab, cfg.width, cfg.side_dim, cfg.logit_softcap, cfg.norm_eps) == (130, 96, 4, 12.0, 3e-4)
    assert [L.type for L in cfg.layers] == ["mamba1", "parallel", "mamba1"] and cfg.layers[1].mlp is None
    assert cfg.layers[1].mixer.left.mask_size == 24 and cfg.layers[1].mixer.right.conv == 4
    assert TibepelConfig.from_dict(cfg.to_dict()) == cfg
    assert resolve_architecture(plain.TINY_Q).name == "Tibepel"
    assert resolve_architecture({"architectures": ["Tibepel"]}).name == "Tibepel"


@pytest.mark.parametrize("change", [
    lambda c: c.pop("vocab"), lambda c: c["layers"][0].update(type="mamba9"), lambda c: c["layers"][1]["mixer"]["left"].update(heads=5),
    lambda c: c["layers"][0]["mlp"].update(kind="sparse"), lambda c: c.update(width=95), lambda c: c["norm"].update(eps=0),
    lambda c: c["layers"][1]["mixer"].pop("left_scale"), lambda c: c.update(layers=[]),
])
def test_config_names_what_is_wrong(change):
    bad = copy.deepcopy(plain.TINY_Q)
    change(bad)
    with pytest.raises(ConfigError):
        TibepelConfig.from_dict(bad)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_the_model_expects_the_checkpoint_names_and_shapes(name):
    from pytriton_llama_b200.models.decoder import DecoderModel
    from pytriton_llama_b200.parts.base import Runtime
    arch = resolve_architecture(plain.TINY[name])
    model = DecoderModel(arch.spec_from_config(arch.config_from_dict(plain.TINY[name])), Runtime(torch.device("cpu"), torch.float32, None))
    assert {k: tuple(v.shape) for k, v in model.expected_tensors().items()} == plain.tensor_shapes(plain.TINY[name])


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from pytriton_llama_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", plain.TINY_P, seed=3, dtype=torch.float32)
    eng = _engine(folder, 4, 32)
    out = eng.step([StepEntry("a", [1, 2, 3, 4, 5], [4])])
    ref = _reference(folder, {"a": [1, 2, 3, 4, 5]})["a"]
    assert torch.isfinite(out.logits).all() and (out.logits[0].double() - ref[4]).abs().max() < TOL


# ---------------------------------------------------------------------------- the cache
def test_pages_before_the_block_of_the_next_query_are_given_back():
    need = CacheNeed(kind="chunk", kv_heads=1, head_dim=4, window=8, value_dim=6, states=(("s", (2, 3)),))
    cache = CacheManager({0: need}, page_size=4, num_pages=6, max_requests=2, max_seq_len=64, device="cpu", dtype=torch.float32)
    assert cache.groups[0].kv[0].shape == (6, 1 * 4 * (4 + 6)) and cache.groups[0].states[0]["s"].shape == (2, 2, 3)
    cache.admit("a")
    cache.append("a", 7)                      # positions 0..6: pages 0, 1
    assert cache.free_pages() == 4
    cache.append("a", 1)                      # position 7 is still in block 0
    assert cache.free_pages() == 4 and cache.block_table("a", 0)[:2] != [-1, -1]
    cache.append("a", 1)                      # position 8 opens block 1: the two pages of block 0 come back first
    assert cache.block_table("a", 0)[:2] == [-1, -1] and cache.free_pages() == 5
    cache.append("a", 11)                     # up to position 19: blocks 1 and 2 (the portion's own queries need block 1)
    assert cache.free_pages() == 3
    cache.append("a", 1)                      # position 20 lies in block 2: block 1's pages go
    assert cache.block_table("a", 0)[:4] == [-1, -1, -1, -1]
    cache.check_invariants()
    cache.release("a")
    assert cache.free_pages() == 6 and cache.free_slots() == 2


# ---------------------------------------------------------------------------- every cut against the whole sequence
@pytest.mark.parametrize("name,page", [("P", 4), ("P", 16), ("Q", 16), ("Q", 8)])
def test_every_cut_gives_the_whole_sequence_logits(folders, name, page):
    folder = folders(name)
    vocab = plain.TINY[name]["vocab"]
    lens = [1, 9, 33, 70, 12, 27]            # six requests through four slots: slots and pages are used again
    seqs = {f"r{i}": random_tokens(n, vocab, 500 + i) for i, n in enumerate(lens)}
    ref = _reference(folder, seqs)
    for family in (traces.whole, traces.prefill_then_decode, traces.portions, traces.mixed):
        steps = family(seqs)
        pages = -(-traces.max_live_tokens(steps, max(page, 8)) // page)
        eng = _engine(folder, page, pages)
        got = traces.replay(eng, steps)
        for r in seqs:
            assert (got[r].double() - ref[r]).abs().max() < TOL, (family.__name__, r)
        assert eng.cache.free_slots() == 4 and all(eng.cache.free_pages(g) == pages for g in eng._paged_groups())


def _single(kind):
    """One-layer models in which one mechanism works alone."""
    a, b = plain.left(4, 2, 16, 8, 8, 0.25), plain.right(4, 2, 8, 16, 3)
    layers = {"scan": plain.layer("mamba1", plain.scan(40, 7, 4, 4), None),
              "attention": plain.layer("parallel", plain.parallel(a, b, 1.0, 0.0), None),
              "delta": plain.layer("parallel", plain.parallel(a, b, 0.0, 1.0), None),
              "feed_forward": plain.layer("parallel", plain.parallel(a, b, 0.0, 0.0), plain.dense(48, 0.8))}
    return plain.config(64, 48, 1, [layers[kind]], scale=1.0, cap=15.0)


@pytest.mark.parametrize("kind", ["scan", "attention", "delta", "feed_forward"])
def test_each_mechanism_alone(folders, kind):
    folder = folders(kind, _single(kind), seed=5)
    seqs = {"a": random_tokens(45, 64, 1), "b": random_tokens(19, 64, 2)}
    ref = _reference(folder, seqs)
    for family in (traces.whole, traces.portions, traces.mixed):
        got = traces.replay(_engine(folder, 4, 40), family(seqs))
        for r in seqs:
            assert (got[r].double() - ref[r]).abs().max() < TOL, (kind, family.__name__, r)


def test_a_model_without_pages(folders):
    """Only selective-scan layers: no keys and values at all, states alone."""
    cfg = plain.config(50, 32, 2, [plain.layer("mamba1", plain.scan(24, 4, 2, 3), plain.dense(40, 2.0)),
                                   plain.layer("mamba1", plain.scan(40, 9, 5, 4), None)], scale=1.5)
    folder = folders("scans", cfg, seed=9)
    seqs = {"a": random_tokens(37, 50, 1), "b": random_tokens(8, 50, 2), "c": random_tokens(21, 50, 3)}
    ref = _reference(folder, seqs)
    for family in (traces.whole, traces.portions, traces.mixed):
        got = traces.replay(_engine(folder, 4, 8, slots=2), family(seqs, live=2) if family is traces.mixed else family(seqs))
        for r in seqs:
            assert (got[r].double() - ref[r]).abs().max() < TOL, (family.__name__, r)


def test_batches_of_unequal_requests_against_each_alone(folders):
    folder = folders("P")
    seqs = {"long": random_tokens(61, 96, 7), "short": random_tokens(3, 96, 8), "one": random_tokens(1, 96, 9)}
    alone = {r: traces.replay(_engine(folder, 4, 40), traces.whole({r: s}))[r] for r, s in seqs.items()}
    eng = _engine(folder, 4, 40)
    out = eng.step([StepEntry(r, s, list(range(len(s)))) for r, s in seqs.items()])
    at = 0
    for r, s in seqs.items():
        assert (out.logits[at:at + len(s)] - alone[r]).abs().max() < 1e-5, r
        at += len(s)


def test_long_decoding_token_by_token(folders):
    folder = folders("Q")
    toks = random_tokens(150, 130, 21)
    ref = _reference(folder, {"a": toks})["a"]
    eng = _engine(folder, 16, 12)
    rows = [eng.step([StepEntry("a", [t], [0])]).logits[0] for t in toks]     # from the first token on, across six blocks
    assert (torch.stack(rows).double() - ref).abs().max() < TOL
    assert eng.cache.free_pages(eng._paged_groups()[0]) >= 12 - 3             # earlier blocks' pages have come back


def test_greedy_generation_through_the_scheduler(folders):
    from pytriton_llama_b200.engine.llm import LLM
    from pytriton_llama_b200.sampling.params import SamplingParams
    folder = folders("P")
    prompts = [random_tokens(n, 96, 40 + i) for i, n in enumerate([5, 23, 2, 14, 9])]
    cfg = EngineConfig(dtype="float32", page_size=4, max_gpu_num_blocks=40, max_seq_len=64, max_num_seqs=3,
                       max_batched_tokens=16, overlap_steps=False)
    outs = LLM(folder, cfg, device="cpu", ops=TorchOps()).generate(prompts, SamplingParams(temperature=0.0, max_gen_len=7))
    W = json.loads((folder / "config.json").read_text())
    for p, o in zip(prompts, outs):
        assert len(o) == 7
        logits = _reference(folder, {"x": p + o})["x"]
        for i, tok in enumerate(o):
            row = logits[len(p) + i - 1]
            assert row[tok] >= row.max() - 1e-3, (i, tok, int(row.argmax()))
