"""Famupel on the host side, without a GPU: its configuration (every key read, faults named, the rank that only a
tensor's shape gives), its weights, the model as data (blocks over streams or over one residual row, what each mixer
keeps), and the whole path through cache manager, step function and replay on the CPU with the kernels replaced by
their PyTorch statements."""
import copy
import io
import json

import numpy as np
import pytest
import torch

import plain_famupel as plain
import replay_cases as rc


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
  return plain.make_model_dir(plain.CONFIGS["A"], str(tmp_path_factory.mktemp("famupel_A")), seed=3, ranks=plain.RANKS["A"])


def test_configuration_is_read_key_by_key(model_a):
  from miniinfer_b200.config import FamupelConfig, load_model_config
  cfg = load_model_config(model_a)
  assert isinstance(cfg, FamupelConfig)
  assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.streams) == (300, 64, 1e-5, 3)
  g, (left, right, ls, rs) = cfg.mixer_of(0), cfg.mixer_of(1)
  assert (g.heads, g.dim, g.vdim, g.tau) == (3, 20, 24, 8.0)
  assert (left.heads, left.kv_heads, left.dim, left.vdim, left.scale, left.rot.dims, left.rot.base) == (4, 1, 24, 16, 0.3, 16, 10000.0)
  assert left.rot.scaling == {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64.0}
  assert (right.heads, right.dim, right.vdim, right.decay, right.rot.dims, right.rot.scaling) == (2, 24, 40, [0.9, 0.996], 8, None)
  assert (ls, rs) == (0.7, 1.3)
  assert [cfg.ff_of(i) for i in range(5)] == [96, 80, None, None, 72]
  # the rank of a decay's projection stands in no key: it is read from the shapes of the file's tensors
  assert cfg.low_ranks == {"l0.decay": 8, "l2.decay": 4, "l4.decay": 16}
  d = cfg.to_dict()
  d.pop("low_ranks")
  assert d == plain.CONFIGS["A"]
  assert FamupelConfig.from_dict(plain.CONFIGS["B"]).streams is None


@pytest.mark.parametrize("change,key", [
  (lambda c: c["layers"][0].__setitem__("type", "attention"), "layers[0].type"),
  (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "left.heads"),
  (lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 30), "rot.dims"),
  (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].__setitem__("factor", 0), "scaling.factor"),
  (lambda c: c["layers"][1]["mixer"]["left"]["rot"]["scaling"].__setitem__("high", 1.0), "scaling.high"),
  (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5]), "right.decay"),
  (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("decay", [0.5, 1.5]), "right.decay"),
  (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
  (lambda c: c["layers"][1]["mixer"].pop("right"), "'left' and 'right'"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("tau", 0), "mixer.tau"),
  (lambda c: c["layers"][0]["mixer"].__setitem__("vdim", 0), "mixer.vdim"),
  (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "moe"), "mlp.kind"),
  (lambda c: c.__setitem__("streams", 0), "streams"),
  (lambda c: c["norm"].__setitem__("eps", 0), "norm.eps"),
  (lambda c: c.__setitem__("width", 0), "width"),
  (lambda c: c.__setitem__("layers", []), "layers"),
])
def test_faulty_configurations_are_refused_with_the_key(change, key):
  from miniinfer_b200.config import ConfigError, FamupelConfig
  c = copy.deepcopy(plain.CONFIGS["A"])
  change(c)
  with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]").replace(".", r"\.")):
    FamupelConfig.from_dict(c)


def test_the_model_as_data(model_a, tmp_path):
  from miniinfer_b200.cache.specs import CompositeSpec, FixedStateSpec, PagedKVSpec
  from miniinfer_b200.config import build_model_spec, load_model_config
  spec = build_model_spec(load_model_config(model_a))
  assert [type(b).__name__ for b in spec.blocks] == ["HyperConnectionBlock"] * 5 and type(spec.final_norm).__name__ == "StreamSumNorm"
  assert [type(b.mixer_part()).__name__ for b in spec.blocks] == ["LinearAttentionMixer", "SideBySideMixer"] * 2 + ["LinearAttentionMixer"]
  assert spec.blocks[2].ffn is None and spec.blocks[2].ffn_norm is None and spec.blocks[0].ffn_norm is not None
  assert spec.embedding.copies == 3
  needs = spec.cache_layer_specs()
  assert needs[0] == FixedStateSpec((3 * 20 * 24,), "float32") and needs[2] == FixedStateSpec((40 * 16,), "float32")
  # keys of 24 and values of 16 share cache rows of 32; all earlier tokens stay (no window)
  assert needs[1] == CompositeSpec((PagedKVSpec(1, 32, None), FixedStateSpec((2 * 24 * 40,), "float32")))
  assert needs[3] == CompositeSpec((PagedKVSpec(2, 32, None), FixedStateSpec((3 * 16 * 8,), "float32")))
  gl, side = spec.blocks[0].mixer_part(), spec.blocks[1].mixer_part()
  assert (gl.decay, gl.decay_rank, gl.tau, gl.q_scale, gl.k_scale, gl.norm_weight, gl.gate) == ("channel", 8, 8.0, 20 ** -0.5, 1.0, True, "silu")
  assert (side.normed, side.left_scale, side.right_scale) == (False, 0.7, 1.3)
  assert (side.left.biases, side.left.norm_whole, side.left.gated, side.left.sinks, side.left.window, side.left.scale) == (True, True, True, False, None, 0.3)
  r = side.right
  assert (r.decay, r.head_decay_values, r.q_scale, r.k_scale, r.norm_weight, r.position.rotary_dim) == ("head", [0.9, 0.996], 1.0, 24 ** -0.5, False, 8)
  # without streams: the usual pre-norm block and a plain final norm
  b = plain.make_model_dir(plain.CONFIGS["B"], str(tmp_path / "B"), seed=1, ranks=plain.RANKS["B"])
  spec_b = build_model_spec(load_model_config(b))
  assert [type(x).__name__ for x in spec_b.blocks] == ["PreNormBlock"] * 3 and type(spec_b.final_norm).__name__ == "RMSNorm"
  assert spec_b.embedding.copies == 1 and spec_b.blocks[2].ffn is None


def test_band_scaled_frequencies():
  """All three bands occur: a frequency that stays, two that are blended, the rest divided by the factor."""
  from miniinfer_b200.parts import BandScaledRotaryEncoding
  rot = plain.CONFIGS["A"]["layers"][1]["mixer"]["left"]["rot"]
  want = plain.rotary_frequencies(rot)
  plain_f = rot["base"] ** (-2.0 * torch.arange(8, dtype=torch.float64) / 16)
  ratio = want / plain_f
  assert ratio[0] == 1.0 and all(1 / 8 < float(r) < 1 for r in ratio[1:3]) and torch.allclose(ratio[3:], torch.full((5,), 1 / 8, dtype=torch.float64))
  pe = BandScaledRotaryEncoding("rot", rot["dims"], rot["base"], 1 << 20, scaling=rot["scaling"])
  assert torch.allclose(pe.frequencies(), want, rtol=1e-14, atol=0)
  table = pe.build_table(200)
  a = torch.arange(200, dtype=torch.float64)[:, None] * want[None]
  assert table.shape == (200, 16) and torch.equal(table, torch.cat((a.cos(), a.sin()), -1).float())
  assert torch.equal(BandScaledRotaryEncoding("rot", 16, 10000.0, 1 << 20).frequencies(), plain_f)


def test_weights_are_asked_for_by_name(model_a, tmp_path):
  from safetensors.torch import load_file, save_file
  from miniinfer_b200.config import build_model_spec, load_model_config
  from miniinfer_b200.weights import load_weights
  from miniinfer_b200.weights.loader import WeightLoadError
  spec = build_model_spec(load_model_config(model_a))
  load_weights(spec, model_a, torch.bfloat16, "cpu")
  W = plain.read_weights(model_a)
  blk = spec.blocks[0]
  assert blk.mixer_norm.weight.dtype == torch.float32 and torch.equal(blk.mixer_norm.weight, W["l0.norm1"])
  assert torch.equal(blk.hc1_mix, W["l0.hc1.mix"]) and torch.equal(blk.hc2_in, W["l0.hc2.in"]) and blk.hc2_out.dtype == torch.float32
  gl = blk.mixer_part()
  assert gl.proj.shape == (8 + 2 * 60 + 2 * 72, 64) and torch.equal(gl.proj[:8].float(), W["l0.mix.a1"])
  assert torch.equal(gl.proj[gl.k_off:gl.v_off].float(), W["l0.mix.k"]) and torch.equal(gl.proj[gl.g_off:].float(), W["l0.mix.g"])
  assert torch.equal(gl.a2_bias, W["l0.mix.a2.b"]) and gl.a2_bias.dtype == torch.float32 and torch.equal(gl.norm, W["l0.mix.norm"])
  side = spec.blocks[1].mixer_part()
  left, right = side.left, side.right
  assert left.qkvg.shape == (4 * 24 + 24 + 16 + 4 * 16, 64) and torch.equal(left.q_norm, W["l1.mix.left.q.norm"]) and left.k_norm.shape == (24,)
  assert torch.equal(left.bias, torch.cat([W["l1.mix.left.q.b"], W["l1.mix.left.k.b"], W["l1.mix.left.v.b"]]))
  assert right.proj.shape == (2 * 2 * 24 + 2 * 2 * 40, 64) and not hasattr(right, "a2") and not side.param_specs()
  assert not hasattr(spec.blocks[2], "hc2_in")           # a layer without a feed-forward has one set of stream weights
  t = load_file(f"{model_a}/model.safetensors")
  del t["l1.mix.left.k.b"]
  t["l2.norm2"] = torch.zeros(64)                         # tolerated: what the absent feed-forward's sublayer would read
  t["l2.mlp.up"] = torch.zeros(8, 64)                     # not tolerated
  t["l0.mix.a2"] = torch.zeros((60, 7))
  d = tmp_path / "broken"
  d.mkdir()
  save_file(t, str(d / "model.safetensors"))
  (d / "config.json").write_text(json.dumps(plain.CONFIGS["A"]))
  with pytest.raises(WeightLoadError) as e:
    load_weights(build_model_spec(load_model_config(str(d))), str(d), torch.bfloat16, "cpu")
  assert e.value.missing == ["l1.mix.left.k.b"] and e.value.unexpected == ["l2.mlp.up"] and "l0.mix.a2" in e.value.wrong_shape[0]


def test_random_weights_mode_writes_a_model_of_the_design(tmp_path):
  from miniinfer_b200.weights import write_random_model
  c = copy.deepcopy(plain.CONFIGS["C"])
  c["low_ranks"] = {"l0.decay": 12}
  d = write_random_model(c, str(tmp_path / "m"), seed=4)
  W, cfg = plain.read_weights(d), plain.read_config(d)
  assert W["l0.mix.a1"].shape == (12, 128) and W["l0.mix.a2"].shape == (160, 12) and W["l1.hc2.mix"].shape == (1, 1)
  assert float(W["l0.mix.a2.b"].mean()) > 1.0 and abs(float(W["l1.hc1.mix"][0, 0]) - 1.0) < 0.2
  assert torch.isfinite(plain.forward(cfg, W, [1, 2, 3])).all()


@pytest.mark.parametrize("tag,page", [("A", 16), ("B", 8), ("C", 64)])
def test_every_cut_gives_the_plain_logits_on_the_host_path(cpu_kernels, tmp_path, tag, page):
  from miniinfer_b200.engine.replay import TraceRunner
  cfg = plain.CONFIGS[tag]
  d = plain.make_model_dir(cfg, str(tmp_path / tag), seed=8, ranks=plain.RANKS[tag])
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
    rc.compare(got, ref, 3e-4, f"famupel {tag}/{name}")
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
  rc.compare(rc.collect(trace, outputs), {rid: plain.forward(cfg, W, ids) for rid, ids in reqs.items()}, 3e-4, "trace program")
