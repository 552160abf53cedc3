"""Luporax on the host side, without a GPU: its configuration (every key read, faults named), its weights (stacked file
tensors, layers that run another layer's weights), the model as data (what each run of a block keeps), and the whole path
through cache manager, step function and replay on the CPU with the kernels replaced by their PyTorch statements."""
import copy
import io
import json

import numpy as np
import pytest
import torch

import plain_luporax as plain
import replay_cases as rc


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
  return plain.make_model_dir(plain.CONFIGS["A"], str(tmp_path_factory.mktemp("luporax_A")), seed=3)


def test_configuration_is_read_key_by_key(model_a):
  from miniinfer_b200.config import LuporaxConfig, load_model_config
  cfg = load_model_config(model_a)
  assert isinstance(cfg, LuporaxConfig)
  assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.residual_mult, cfg.logit_scale) == (300, 64, 1e-5, 0.5, 0.3)
  g, a, r = cfg.mixer_of(0), cfg.mixer_of(1), cfg.mixer_of(2)
  assert g.width == 40
  assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.softcap, a.rot.dims, a.rot.base) == (4, 1, 24, 16, 0.3, 20.0, 16, 10000.0)
  assert (r.width, r.blocks, r.conv) == (48, 3, 3)
  m = cfg.mlp_of(0)
  assert (m.ff, m.limit, m.experts, m.top, m.shared.ff, m.shared.limit) == (24, 1.5, 5, 2, 16, 0.8)
  assert cfg.mlp_of(2) is None
  assert [cfg.weights_layer(i) for i in range(6)] == [0, 1, 2, 1, 2, 1]      # layer 5 names layer 3, which names layer 1
  assert cfg.to_dict() == plain.CONFIGS["A"]
  b = LuporaxConfig.from_dict(plain.CONFIGS["B"])
  assert b.mixer_of(1).softcap is None and b.mlp_of(0).shared is None


@pytest.mark.parametrize("change,key", [
  (lambda c: c["layers"][0].__setitem__("type", "gla"), "layers[0].type"),
  (lambda c: c["layers"][1]["mixer"].__setitem__("kv_heads", 3), "mixer.heads"),
  (lambda c: c["layers"][1]["mixer"]["rot"].__setitem__("dims", 30), "rot.dims"),
  (lambda c: c["layers"][1]["mixer"].__setitem__("softcap", -1.0), "mixer.softcap"),
  (lambda c: c["layers"][1]["mixer"].pop("scale"), "mixer.scale"),
  (lambda c: c["layers"][2]["mixer"].__setitem__("blocks", 5), "mixer.width"),
  (lambda c: c["layers"][2]["mixer"].__setitem__("conv", 0), "mixer.conv"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("width", 0), "mixer.width"),
  (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "dense"), "mlp.kind"),
  (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "router.top"),
  (lambda c: c["layers"][0]["mlp"]["expert"].__setitem__("limit", 0), "expert.limit"),
  (lambda c: c["layers"][0]["mlp"]["shared"].pop("ff"), "shared.ff"),
  (lambda c: c["layers"][3].__setitem__("weights_of", 7), "weights_of"),
  (lambda c: c["layers"][1].__setitem__("weights_of", 3), "weights_of"),
  (lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 32), "differs"),
  (lambda c: c.__setitem__("residual_mult", None), "residual_mult"),
  (lambda c: c.pop("logit_scale"), "logit_scale"),
  (lambda c: c["norm"].__setitem__("eps", 0), "norm.eps"),
  (lambda c: c.__setitem__("width", 0), "width"),
  (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_faulty_configurations_are_refused_with_the_key(change, key):
  from miniinfer_b200.config import ConfigError, LuporaxConfig
  c = copy.deepcopy(plain.CONFIGS["A"])
  change(c)
  with pytest.raises(ConfigError) as e:
    LuporaxConfig.from_dict(c)
  assert key in str(e.value)


def test_the_model_as_data(model_a):
  from miniinfer_b200.cache.specs import CompositeSpec, FixedStateSpec, PagedKVSpec
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.parts import GatedAttentionMixer, MinGruMixer, OutputNormBlock, RglruMixer, RoutedExpertsFeedForward
  spec = build_model_spec(load_model_config(model_a))
  # three blocks own tensors; six runs, every one with a cache and a state of its own
  assert len(spec.blocks) == 3 and [r.block for r in spec.run_list] == [0, 1, 2, 1, 2, 1]
  assert all(r.cache_of is None for r in spec.run_list)
  assert [type(b.mixer) for b in spec.blocks] == [MinGruMixer, GatedAttentionMixer, RglruMixer]
  assert all(isinstance(b, OutputNormBlock) and b.token_shift and b.mult == 0.5 for b in spec.blocks)
  att = spec.blocks[1].mixer
  assert att.sigmoid_weights and att.softcap == 20.0 and att.biases and att.norm_whole and not att.sinks and not att.gated
  ff = spec.blocks[0].ffn
  assert isinstance(ff, RoutedExpertsFeedForward) and spec.blocks[2].ffn is None
  assert (ff.router_weights, ff.activation, ff.limit, ff.shared_size, ff.shared_limit, ff.shared_gate) == ("softmax_chosen", "clamped", 1.5, 16, 0.8, True)
  shift = FixedStateSpec((64,), "float32")
  specs = spec.cache_layer_specs()
  assert specs[0] == CompositeSpec((shift, FixedStateSpec((40,), "float32")))
  assert specs[1] == specs[3] == specs[5] == CompositeSpec((shift, PagedKVSpec(1, 32, None, 0)))        # rows of max(dim, vdim), padded to 16
  assert specs[2] == specs[4] == CompositeSpec((shift, FixedStateSpec((2 * 48 + 48,), "float32")))      # two earlier inputs of the convolution, then the state
  assert spec.final_norm.offset == 1.0 and spec.final_norm.gain == 0.3 and spec.lm_head.tied_to is spec.embedding


def test_weights_are_asked_for_by_name(model_a, tmp_path):
  from safetensors.torch import load_file, save_file
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.weights import WeightLoadError, load_weights
  spec = build_model_spec(load_model_config(model_a))
  load_weights(spec, model_a, torch.float32, "cpu")
  W = plain.read_weights(model_a)
  r = spec.blocks[2].mixer
  # the gates of a part stand side by side: rows of Ra, then of Ri, part after part; their biases one a channel
  assert torch.equal(r.gates.view(3, 32, 16)[1, :16], W["l2.mix.ra"][1]) and torch.equal(r.gates.view(3, 32, 16)[2, 16:], W["l2.mix.ri"][2])
  assert torch.equal(r.ra_b, W["l2.mix.ra.b"].reshape(-1)) and torch.equal(r.w_in[:48], W["l2.mix.x"]) and torch.equal(r.w_in[48:], W["l2.mix.y"])
  ff = spec.blocks[0].ffn
  assert torch.equal(ff.router[:5], W["l0.mlp.router"]) and torch.equal(ff.router[5:], W["l0.mlp.shared.sg"])
  assert torch.equal(spec.blocks[1].norm1.weight if hasattr(spec.blocks[1], "norm1") else spec.blocks[1].mixer_norm.weight, 1.0 + W["l1.norm1"])
  assert torch.allclose(spec.final_norm.weight, (1.0 + W["final.norm"]) * 0.3)
  raw = load_file(f"{model_a}/model.safetensors")
  raw.pop("l1.mix.pb")
  raw["l3.shift"] = raw["l1.shift"].clone()                   # a layer that runs another's weights has none of its own
  raw["l2.mix.ra"] = raw["l2.mix.ra"][:, :, :8].contiguous()
  d = tmp_path / "broken"
  d.mkdir()
  (d / "config.json").write_text(json.dumps(plain.CONFIGS["A"]))
  save_file(raw, str(d / "model.safetensors"))
  with pytest.raises(WeightLoadError) as e:
    load_weights(build_model_spec(load_model_config(str(d))), str(d), torch.bfloat16, "cpu")
  assert e.value.missing == ["l1.mix.pb"] and e.value.unexpected == ["l3.shift"] and "l2.mix.ra" in e.value.wrong_shape[0]


def test_random_weights_mode_writes_a_model_of_the_design(tmp_path):
  from miniinfer_b200.weights import write_random_model
  d = write_random_model(copy.deepcopy(plain.CONFIGS["B"]), str(tmp_path / "m"), seed=4)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  assert set(W) == set(plain.tensor_shapes(plain.CONFIGS["B"])) and all(tuple(W[k].shape) == s for k, s in plain.tensor_shapes(plain.CONFIGS["B"]).items())
  assert float(W["l0.mix.ra"].abs().sum()) > 0 and torch.isfinite(plain.forward(cfg, W, [1, 2, 3])).all()


@pytest.mark.parametrize("tag,page", [("A", 16), ("B", 8), ("C", 64), ("D", 16)])
def test_every_cut_gives_the_plain_logits_on_the_host_path(cpu_kernels, tmp_path, tag, page):
  from miniinfer_b200.engine.replay import TraceRunner
  cfg = plain.CONFIGS[tag]
  d = plain.make_model_dir(cfg, str(tmp_path / tag), seed=8)
  lengths = (5, 17, 33, 70, 64, 41, 2, 1)
  reqs = rc.make_requests(cfg["vocab"], lengths, seed=5)
  W = plain.read_weights(d)
  ref = {rid: plain.forward(cfg, W, ids) for rid, ids in reqs.items()}
  budget = 2 * rc.round_up(max(lengths), page)
  for name, trace in (("whole", rc.whole(reqs)), ("tail", rc.tail_one_by_one(reqs)), ("portions", rc.portions(reqs)),
                      ("mixed", rc.mixed(reqs, budget, seed=1, granule=page)),
                      ("preempted", rc.mixed(reqs, budget, seed=2, granule=page, preempt=True))):
    runner = TraceRunner(d, "float32", budget, device="cpu", page_size=page, max_requests=4)
    got = rc.run_in_process(runner, trace)
    rc.compare(got, ref, 1e-3, f"luporax {tag}/{name}")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == [g.num_pages for g in runner.cache.paged_groups]


def test_trace_program_picks_the_model_by_its_configuration(cpu_kernels, model_a, tmp_path):
  from miniinfer_b200.engine import replay
  reqs = rc.make_requests(300, (20, 9), seed=2)
  trace = rc.mixed(reqs, 128, seed=3)
  out = io.StringIO()
  code = replay.main(["--model", model_a, "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128",
                      "--device", "cpu"], stdin=io.StringIO("\n".join(json.dumps(r) for r in trace) + "\n"), stdout=out)
  assert code == 0 and out.getvalue().split("\n")[:-1] == [f"done {r['step']}" for r in trace]
  outputs = {r["step"]: np.fromfile(tmp_path / "o" / f"{r['step']}.f32", dtype="<f4").reshape(-1, 300)
             for r in trace if sum(len(e["want"]) for e in r["entries"])}
  W, cfg = plain.read_weights(model_a), plain.read_config(model_a)
  rc.compare(rc.collect(trace, outputs), {rid: plain.forward(cfg, W, ids) for rid, ids in reqs.items()}, 1e-3, "trace program")
