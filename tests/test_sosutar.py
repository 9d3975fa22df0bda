"""Sosutar on the host side: configuration, spec, random weights, state rows, and the step function,
batching and generation loop over the CPU double of the kernels, against the plain implementation."""
import json

import numpy as np
import pytest
import torch

import ember_cpp_b200 as E
from ember_cpp_b200.config import ConfigError, SosutarConfig, config_from_dict
from ember_cpp_b200.parts import DecoderModel
from ember_cpp_b200.weights import read_folder

import plain_sosutar as P
import sosutar_util as U
from conftest import run_batch
from cpu_ops import CpuOps


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: U.write_model(str(tmp_path_factory.mktemp(name)), U.config(name), U.SEEDS[name]) for name in U.CONFIGS}


@pytest.fixture(scope="module")
def plains(folders):
    return {name: P.PlainSosutar(folder) for name, folder in folders.items()}


def cpu_engine(folder, max_tokens=1024, dtype="float32"):
    return E.Engine.from_folder(folder, dtype=dtype, max_tokens=max_tokens, device="cpu", ops=CpuOps())


# ------------------------------------------------------------------------------ configuration
def test_the_architecture_is_registered_and_reads_its_own_keys():
    cfg = config_from_dict(U.config("sos_a"))
    assert isinstance(cfg, SosutarConfig) and "Sosutar" in E.config.architectures()
    assert (cfg.vocab, cfg.width, cfg.max_positions, cfg.norm_eps, cfg.embedding_scale, cfg.logit_scale, len(cfg.layers)) == \
        (300, 64, 700, 1e-5, 4.0, 0.25, 5)
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("path, value, word", [
    (("width",), None, "width"), (("norm", "eps"), 0, "norm.eps"), (("layers", 0, "type"), "serial", "type"),
    (("max_positions",), 0, "max_positions"), (("embedding", "scale"), None, "embedding.scale"),
    (("layers", 1, "mixer", "left", "mask", "size"), 0, "mask.size"), (("layers", 0, "mixer", "gate_cap"), None, "gate_cap"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "kv_heads"), (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("layers", 1, "mixer", "right", "width"), 0, "right.width"), (("layers", 1, "mixer", "left", "q_temp", "every"), 0, "every"),
    (("layers", 2, "weights_of"), 2, "weights_of"), (("layers", 2, "weights_of"), 1, "weights_of"),
    (("layers", 4, "weights_of"), 2, "weights_of")])
def test_a_bad_value_is_refused_by_its_key(path, value, word):
    d = U.config("sos_a")
    at = d
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        config_from_dict(d)


def test_a_layer_that_runs_with_another_layers_tensors_is_an_entry_of_the_run_order():
    """It has no tensors and no parts of its own, and state and cache of its own; the other layer may come later."""
    for name, layers, order in (("sos_a", 3, [0, 1, 0, 2, 1]), ("sos_b", 2, [1, 0, 1])):
        cfg = config_from_dict(U.config(name))
        spec = E.config.get_architecture("Sosutar").build_spec(cfg)
        assert len(spec.layers) == layers and [a.layer for a in spec.schedule] == order
        assert all(a.cache_of is None for a in spec.schedule)
        model = DecoderModel(spec)
        names = [w.name for w in model.weight_specs()]
        assert len(names) == len(set(names))
        owners = {n.split(".")[0] for n in names if n.startswith("l")}
        assert owners == {f"l{i}" for i, layer in enumerate(cfg.layers) if "weights_of" not in layer}
        needs = model.application_needs()
        assert len(needs) == len(cfg.layers)
        for (cache, state), layer in zip(needs, cfg.layers):
            if layer["type"] == "mlstm":
                assert cache is None and set(state) == {"S", "n", "m"}
            else:
                assert cache.kind == "window" and cache.window == layer["mixer"]["left"]["mask"]["size"]
                assert set(state) == {"right."} and state["right."].shape == (layer["mixer"]["right"]["width"],)
    assert spec.scale_positions is False and spec.logit_scale == 2.0 and spec.embedding_scale == 0.5
    # a layer may name a layer that names a third: all three run with the third's tensors
    d = U.config("sos_a")
    d["layers"].append(dict(d["layers"][2], weights_of=2))
    cfg = config_from_dict(d)
    spec = E.config.get_architecture("Sosutar").build_spec(cfg)
    assert [a.layer for a in spec.schedule] == [0, 1, 0, 2, 1, 0] and cfg.owner_of(5) == 0
    d["layers"][0] = dict(d["layers"][0], weights_of=5)         # ... but not in a ring
    with pytest.raises(ConfigError, match="weights_of"):
        config_from_dict(d)


def test_random_weights_follow_the_parts_lists(folders):
    t = read_folder(folders["sos_a"])
    assert t["l0.mix.i.b"].shape == (2,) and t["l1.mix.left.sink"].shape == (4,) and t["l1.mix.left.q.norm"].shape == (64,)
    assert t["l1.mix.right.z"].shape == (40, 64) and t["l1.ls2"].shape == (64,) and t["pos"].shape == (700, 64)
    assert not any(n.startswith(("l2.", "l4.")) for n in t) and "l3.ls2" not in t and "l3.norm2" not in t


# ------------------------------------------------------------------------------ the step function over the double
@pytest.mark.parametrize("name", ["sos_a", "sos_b", "sos_c"])
def test_prompts_decoding_portions_and_batches_equal_the_plain_model(folders, plains, name):
    eng, m = cpu_engine(folders[name]), plains[name]
    vocab = m.cfg["vocab"]
    seqs = [U.ids(10 + i, vocab, n) for i, n in enumerate((70, 1, 23, 2))]
    refs = [P.forward(m, s) for s in seqs]
    for prompts in ([len(s) for s in seqs], [40, 1, 1, 1]):
        got, _ = run_batch(eng, seqs, prompts)
        assert max(U.row_error(g, r) for g, r in zip(got, refs)) < U.TOL["float32"]
    slot, at, rows = eng.open(), 0, []
    for n in (2, 5, 30, 3, 2, 28):                                                 # portions of one sequence
        rows.append(eng.step([(slot, seqs[0][at:at + n], list(range(n)))]).numpy())
        at += n
    eng.close(slot)
    assert U.row_error(np.concatenate(rows), refs[0]) < U.TOL["float32"]
    eng.cache.check()
    assert eng.cache.slots.held == 0 and all(g.pages.held == 0 for g in eng.cache.groups)


def test_state_rows_and_pages_are_used_again(folders, plains):
    """A small cache: the next batch gets the slots, state rows and pages that the batch before it left
    (filled with NaN in between); a sequence that begins must not read them."""
    eng, m = cpu_engine(folders["sos_a"], max_tokens=256), plains["sos_a"]
    for round_ in range(2):
        seqs = [U.ids(200 * round_ + i, 300, n) for i, n in enumerate((100, 30))]
        got, slots = run_batch(eng, seqs, [3, 25])
        assert sorted(slots) == [0, 1]
        assert max(U.row_error(g, P.forward(m, s)) for g, s in zip(got, seqs)) < U.TOL["float32"]
        for g in eng.cache.groups:
            for t in g.k + g.v:
                t.fill_(float("nan"))
        for state in eng.cache.states:
            for t in state.values():
                t.fill_(float("nan"))


def test_the_position_table_bounds_the_context(folders):
    eng = cpu_engine(folders["sos_c"], max_tokens=1024)
    slot = eng.open()
    with pytest.raises(E.StepError, match="position"):
        eng.step([(slot, [1] * 301, [300])])
    assert eng.step([(slot, [1] * 300, [299])].copy()) is not None


def test_greedy_generation_through_the_session(folders, plains):
    for name in ("sos_a", "sos_b"):
        m = plains[name]
        session = E.Session(folders[name], None, max_batch_size=3, dtype="float32", max_tokens=1024, ops=CpuOps(), device="cpu")
        prompts = [U.ids(50 + i, m.cfg["vocab"], n) for i, n in enumerate((5, 23, 1, 9))]
        assert session.generate_batch(prompts, steps=6, temperature=0.0) == [P.generate(m, p, 6) for p in prompts]


def test_the_command_line_writes_a_random_model_of_this_design(tmp_path):
    from ember_cpp_b200 import cli
    cfg_file = tmp_path / "cfg.json"
    cfg_file.write_text(json.dumps(U.config("sos_b")))
    out = tmp_path / "model"
    assert cli.main([str(out), "-", "1", "random-weights", "--config", str(cfg_file), "--seed", "5"]) == 0
    cfg = E.load_config(str(out))
    assert isinstance(cfg, SosutarConfig) and cfg.width == 96
    eng = cpu_engine(str(out), max_tokens=128)
    slot = eng.open()
    logits = eng.step([(slot, U.ids(1, 200, 9), [8])])
    assert tuple(logits.shape) == (1, 200) and bool(torch.isfinite(logits).all())
