"""Vipolix on the host side: configuration, spec, random weights, the cache's chunk groups, and the step function,
batching and generation loop over the CPU double of the kernels, against the plain implementation."""
import json

import numpy as np
import pytest

import ember_cpp_b200 as E
from ember_cpp_b200.cache.sequence_cache import SequenceCache
from ember_cpp_b200.config import ConfigError, VipolixConfig, config_from_dict
from ember_cpp_b200.parts import CacheNeed, DecoderModel
from ember_cpp_b200.weights import read_folder

import plain_vipolix as P
import vipolix_util as U
from conftest import run_batch
from cpu_ops import CpuOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: U.write_model(str(tmp_path_factory.mktemp(name)), U.config(name), U.SEEDS[name]) for name in U.CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: P.load_folder(folder) for name, folder in folders.items()}


def cpu_engine(folder, max_tokens=1024, dtype="float32"):
    return E.Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, device="cpu", ops=CpuOps())


# ------------------------------------------------------------------------------ configuration
def test_the_architecture_is_registered_and_reads_its_own_keys():
    cfg = config_from_dict(U.config("vip_a"))
    assert isinstance(cfg, VipolixConfig) and "Vipolix" in E.config.architectures()
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.side_dim, len(cfg.layers)) == (300, 64, 1e-5, 8, 4)
    assert config_from_dict(cfg.to_dict()) == cfg
    assert config_from_dict(U.config("vip_b")).side_dim == 0


@pytest.mark.parametrize("path, value, word", [
    (("width",), None, "width"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "serial", "type"),
    (("token_side", "dim"), 0, "token_side.dim"), (("layers", 1, "mixer", "tau"), 0, "tau"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, "mask.size"), (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 7, "rot.dims"), (("layers", 0, "mixer", "left", "rot", "dims"), 34, "rot.dims"),
    (("layers", 0, "mixer", "left", "conv"), None, "conv"), (("layers", 0, "mixer", "right", "heads"), 0, "right.heads"),
    (("layers", 0, "mlp", "kind"), "dense", "kind"), (("layers", 0, "mlp", "router", "top"), 9, "top"),
    (("layers", 0, "mlp", "router", "groups", "count"), 3, "groups"), (("layers", 0, "mlp", "router", "groups", "keep"), 5, "groups"),
    (("layers", 3, "mlp", "router", "groups", "keep"), 0, "keep"), (("layers", 0, "mlp", "shared", "limit"), None, "shared.limit"),
    (("layers", 0, "mlp", "expert", "limit"), -1.0, "expert.limit"), (("layers", 0, "mixer", "left_scale"), None, "left_scale")])
def test_a_bad_value_is_refused_by_its_key(path, value, word):
    d = U.config("vip_a")
    at = d
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_the_spec_wraps_every_mixer_in_a_token_shift_and_names_the_designs_tensors(folders):
    cfg = config_from_dict(U.config("vip_a"))
    spec = E.config.get_architecture("Vipolix").build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["token_shift"] * 4
    assert [l.mixer.params["inner"].kind for l in spec.layers] == ["parallel", "gated_linear_attention"] * 2
    assert spec.layers[1].ffn is None and spec.layers[1].norm2 is None and [len(l.addons) for l in spec.layers] == [1] * 4
    model = DecoderModel(spec)
    needs = model.application_needs()
    assert needs[0][0] == CacheNeed("chunk", 2, 32, 20, 0, 0) and needs[1][0] is None
    assert sorted(needs[0][1]) == ["inner.left.conv", "inner.right.S", "shift"] and sorted(needs[1][1]) == ["inner.S", "shift"]
    assert needs[0][1]["inner.left.conv"].shape == (3, 4 * 32 + 2 * 32 + 2 * 32)
    t = read_folder(folders["vip_a"])
    assert t["l0.shift"].shape == (64,) and t["side.embed"].shape == (300, 32) and t["l0.mix.left.q.conv"].shape == (128, 4)
    assert t["l0.mix.left.temp"].shape == (4,) and t["l0.mix.right.w2"].shape == (32, 16) and t["l3.mix.a1"].shape == (5, 64)
    assert t["l0.mlp.shared.sg"].shape == (1, 64) and t["l0.mlp.correction"].shape == (8,) and "l1.norm2" not in t
    assert "l2.mlp.shared.gate" not in t and t["l1.mix.a2.b"].shape == (32,)
    # the rank of the decays' products is the stored tensors': the same folder loads whatever the configuration says
    d = U.config("vip_a")
    d["layers"][3]["mixer"].pop("decay_rank")
    cpu_engine_of = E.Engine.from_spec(E.config.get_architecture("Vipolix").build_spec(config_from_dict(d)), dict(t),
                                       dtype="float32", max_tokens=128, device="cpu", ops=CpuOps())
    assert cpu_engine_of.model.blocks[3].mixer.inner.rank == 5


def test_a_chunk_group_keeps_the_pages_of_the_querys_own_chunk_alone():
    need = CacheNeed("chunk", 1, 16, 100, 0, 0)
    cache = SequenceCache([(need, None)], [None], 1024, None, __import__("torch").float32, "cpu")
    slot = cache.open()
    cache.reserve([(slot, 250)])
    cache.commit([(slot, 250)])
    held = cache.groups[0].held[slot]
    assert [p >= 0 for p in held] == [False, False, False, True]       # the chunk of position 250 begins at 200: block 3
    cache.reserve([(slot, 60)])
    cache.commit([(slot, 60)])
    assert [p >= 0 for p in cache.groups[0].held[slot]] == [False, False, False, False, True]   # 310 -> 300: block 4
    cache.close(slot)
    cache.check()


def test_the_router_of_the_plain_model_keeps_to_the_best_groups():
    W = {"r.router": np.eye(8) * 4, "r.correction": np.array([0, 0, 0.5, 0.5, 0, 0, -9.0, 3.0])}
    h = np.array([[0.5, 0.5, -0.5, -0.5, -0.5, -0.5, 0.5, 0.5]])
    # scores: sigmoid(+-2); choice adds the correction; groups of two: (0.88, 0.88), (0.62, 0.62), (0.12, 0.12), (-8.1, 3.9)
    chosen, weights = P.route(h, W, "r.", {"experts": 8, "top": 2, "scale": 2.0, "groups": {"count": 4, "keep": 1}})
    assert sorted(chosen[0]) == [0, 1] and np.allclose(weights.sum(), 2.0) and np.allclose(weights[0, 0], 1.0)
    chosen, weights = P.route(h, W, "r.", {"experts": 8, "top": 2, "scale": 1.0})
    assert sorted(chosen[0]) == [0, 7] or sorted(chosen[0]) == [1, 7]
    s = 1 / (1 + np.exp(-2.0))
    assert np.allclose(sorted(weights[0]), [0.5, 0.5]) and np.allclose(P.sigmoid(2.0), s)


# ------------------------------------------------------------------------------ the step function over the double
@pytest.mark.parametrize("name", ["vip_a", "vip_b", "vip_c"])
def test_prompts_decoding_portions_and_batches_equal_the_plain_model(folders, plains, name):
    eng, (cfg, W) = cpu_engine(folders[name]), plains[name]
    seqs = [U.ids(10 + i, cfg["vocab"], n) for i, n in enumerate((75, 1, 23, 2))]
    refs = [P.forward(cfg, W, s) for s in seqs]
    for prompts in ([len(s) for s in seqs], [40, 1, 1, 1]):
        got, _ = run_batch(eng, seqs, prompts)
        assert max(U.row_error(g, r) for g, r in zip(got, refs)) < U.TOL["float32"]
    slot, at, rows = eng.open(), 0, []
    for n in (2, 5, 30, 3, 2, 33):                                                 # portions of one sequence
        rows.append(eng.step([(slot, seqs[0][at:at + n], list(range(n)))]).numpy())
        at += n
    eng.close(slot)
    assert U.row_error(np.concatenate(rows), refs[0]) < U.TOL["float32"]
    eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


def test_the_stream_after_every_layer(folders, plains):
    cfg, W = plains["vip_a"]
    eng = cpu_engine(folders["vip_a"])
    seq = U.ids(77, cfg["vocab"], 31)
    _, streams = P.forward(cfg, W, seq, per_layer=True)
    seen = []
    for block in eng.model.blocks:
        inner = block.forward
        # (a copy: the next layer may add into the stream in place)
        block.forward = lambda ctx, x, app, inner=inner: (lambda y: seen.append(y.clone()) or y)(inner(ctx, x, app))
    slot = eng.open()
    eng.step([(slot, seq, [30])])
    for got, want in zip(seen, streams):
        assert np.abs(got.numpy() - want).max() < 1e-4 * np.abs(want).max()


def test_state_rows_and_pages_are_used_again(folders, plains):
    """A small cache: the next batch gets the slots, state rows and pages that the batch before it left
    (filled with NaN in between); a sequence that begins must not read them."""
    eng, (cfg, W) = cpu_engine(folders["vip_a"], max_tokens=256), plains["vip_a"]
    for round_ in range(2):
        seqs = [U.ids(200 * round_ + i, 300, n) for i, n in enumerate((100, 30))]
        got, slots = run_batch(eng, seqs, [3, 25])
        assert sorted(slots) == [0, 1]
        assert max(U.row_error(g, P.forward(cfg, W, s)) for g, s in zip(got, seqs)) < U.TOL["float32"]
        for g in eng.cache.groups:
            for t in g.k + g.v:
                t.fill_(float("nan"))
        for state in eng.cache.states:
            for t in state.values():
                t.fill_(float("nan"))


def test_greedy_generation_through_the_session(folders, plains):
    for name in ("vip_a", "vip_c"):
        cfg, W = plains[name]
        session = E.Session(folders[name], None, max_batch_size=3, dtype="float32", max_tokens=1024, ops=CpuOps(), device="cpu")
        prompts = [U.ids(50 + i, cfg["vocab"], n) for i, n in enumerate((5, 23, 1, 9))]
        assert session.generate_batch(prompts, steps=6, temperature=0.0) == [P.generate(cfg, W, p, 6) for p in prompts]


def test_the_command_line_writes_a_random_model_of_this_design(tmp_path):
    from ember_cpp_b200 import cli
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(U.config("vip_b")))
    out = tmp_path / "model"
    assert cli.main([str(out), "-", "1", "random-weights", "--config", str(cfg_file), "--seed", "5"]) == 0
    cfg = E.load_config(str(out))
    assert isinstance(cfg, VipolixConfig) and cfg.width == 96
