"""Each mechanism of the Famupel design alone: the engine's operation, run over a step cut in several ways, against the
plain function of tests/plain_famupel.py on the whole sequence.  Inputs are made so that a fault shows: one key far
back whose product with the query stands out, decays of exactly 0 and 1, states of other requests that must be left
alone, sizes that are no powers of two and values that other models happen to make equal or 1."""
from types import SimpleNamespace

import pytest
import torch

import plain_famupel as plain
from gpu_helpers import DEV

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def tol(dtype):
  return 3e-5 if dtype == "float32" else 4e-2


def step_ctx(items):
  """The description of a step: ``items`` = (new tokens, position of the first of them, state slot) for each request."""
  q_len = [n for n, _, _ in items]
  q_start = [sum(q_len[:i]) for i in range(len(q_len))]
  dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
  return SimpleNamespace(q_start=dev(q_start), q_len=dev(q_len), seq_slot=dev([s for _, _, s in items]), num_items=len(items),
                         token_item=dev([b for b, n in enumerate(q_len) for _ in range(n)]),
                         positions=dev([p0 + i for n, p0, _ in items for i in range(n)]))


def cuts_of(T, sizes):
  out, pos, k = [], 0, 0
  while pos < T:
    n = min(sizes[k % len(sizes)], T - pos)
    out.append(n)
    pos += n
    k += 1
  return out


def plain_linear_attention(q, k, v, gate, alpha, eps, rot=None, q_scale=1.0, k_scale=1.0, norm_w=None, silu=True):
  """The whole sequence at once, from the plain pieces: q, k [T, H, D] float32, alpha [T, H, D]; -> [T, H * Dv]."""
  T = q.shape[0]
  if rot is not None:
    pos = torch.arange(T)
    q, k = plain.rotate_half(q, pos, rot), plain.rotate_half(k, pos, rot)
  o = plain.rms_unit(plain.decayed_linear_attention(q * q_scale, k * k_scale, v, alpha), eps)
  if norm_w is not None:
    o = o * norm_w
  g = gate.float().view(o.shape)
  return (o * (plain.silu(g) if silu else torch.sigmoid(g))).reshape(T, -1)


def run_linear_attention(cuts, dtype, q, k, v, gate, H, D, Dv, eps, slot=2, slots=4, pe=None, **kw):
  """One request's tokens in portions ``cuts``; beside it in every step a one-token item of another request in slot 0."""
  from miniinfer_b200.kernels import ops
  T = q.shape[0]
  state = torch.zeros((slots, H * D * Dv + 3), dtype=torch.float32, device=DEV)
  state[1].fill_(7.0)                                   # nobody's slot: to be left alone
  got = torch.zeros((T, H * Dv), dtype=DT[dtype], device=DEV)
  logits = kw.pop("decay_logits", None)
  dev = lambda t: t.to(DEV)
  pos = 0
  for n in cuts:
    rows = torch.cat((torch.arange(pos, pos + n), torch.tensor([0])))
    out = torch.zeros((n + 1, H * Dv), dtype=DT[dtype], device=DEV)
    ops.linear_attention(out, dev(q[rows]), dev(k[rows]), dev(v[rows]), dev(gate[rows]), state, step_ctx([(n, pos, slot), (1, 0, 0)]),
                         H, D, Dv, eps, decay_logits=dev(logits[rows]) if logits is not None else None,
                         rope=pe.rotary_table() if pe is not None else None, **kw)
    got[pos:pos + n] = out[:n]
    pos += n
  assert pos == T
  assert float((state[1] - 7.0).abs().max()) == 0
  return got.float().cpu(), state[slot, :H * D * Dv].cpu().view(H, D, Dv)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,tau", [(2, 16, 24, 8.0), (3, 20, 8, 1.0), (1, 160, 32, 16.0), (4, 64, 64, 4.0), (1, 40, 136, 2.0), (2, 128, 128, 32.0)])
def test_gated_linear_attention_against_the_plain_recurrence(dtype, H, D, Dv, tau):
  g = torch.Generator().manual_seed(H * D + Dv)
  T, eps = 45, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  q, k, v, gate = (r(T, H * n).to(DT[dtype]) for n in (D, D, Dv, Dv))
  logits, bias, norm_w = 2.0 * r(T, H * D), 1.0 + r(H * D), 1 + 0.2 * r(Dv)
  alpha = torch.exp(torch.nn.functional.logsigmoid(logits + bias) / tau).view(T, H, D)
  want = plain_linear_attention(q.float().view(T, H, D), k.float().view(T, H, D), v.float().view(T, H, Dv), gate, alpha, eps,
                                q_scale=D ** -0.5, norm_w=norm_w)
  for sizes in ((T,), (1,), (2,), (2, 7, 1, 33), (17, 16)):
    got, _ = run_linear_attention(cuts_of(T, sizes), dtype, q, k, v, gate, H, D, Dv, eps, decay_logits=logits, decay_bias=bias.to(DEV),
                                  tau=tau, q_scale=D ** -0.5, norm_weight=norm_w.to(DEV))
    assert float((got - want).abs().max()) <= 2 * tol(dtype), f"cut into {sizes}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,rot_dims,decay", [(2, 24, 40, 8, [0.9, 0.996]), (3, 16, 8, 16, [1.0, 0.0, 0.5]), (1, 136, 16, 136, [0.99]),
                                                  (4, 64, 32, 64, [0.96875, 0.995, 0.997, 0.999])])
def test_retention_against_the_plain_recurrence(dtype, H, D, Dv, rot_dims, decay):
  """A constant decay a head - 1 (nothing is forgotten) and 0 (only the token itself is read) among them -, rotated
  queries and keys with positions that go on across the cuts, keys scaled after the rotation, no norm weight."""
  from miniinfer_b200.parts import BandScaledRotaryEncoding
  g = torch.Generator().manual_seed(D + Dv)
  T, eps = 45, 1e-6
  r = lambda *s: torch.randn(s, generator=g)
  q, k, v, gate = (r(T, H * n).to(DT[dtype]) for n in (D, D, Dv, Dv))
  rot = {"dims": rot_dims, "base": 300.0}
  pe = BandScaledRotaryEncoding("rot", rot_dims, 300.0, 4096)
  pe.prepare(DEV, 64)
  alpha = torch.tensor(decay)[None, :, None].expand(T, H, D)
  want = plain_linear_attention(q.float().view(T, H, D), k.float().view(T, H, D), v.float().view(T, H, Dv), gate, alpha, eps, rot=rot,
                                k_scale=D ** -0.5)
  for sizes in ((T,), (1,), (2,), (5, 1, 1, 30)):
    got, _ = run_linear_attention(cuts_of(T, sizes), dtype, q, k, v, gate, H, D, Dv, eps, pe=pe, k_scale=D ** -0.5,
                                  head_decay=torch.tensor(decay, dtype=torch.float32, device=DEV))
    assert float((got - want).abs().max()) <= 2 * tol(dtype), f"cut into {sizes}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("channel", [True, False])
def test_a_key_far_back_is_read_through_the_state(dtype, channel):
  """Token 5 writes a key that no other token's key resembles, 700 tokens before the queries that ask for it; its
  decays are (nearly) 1 on that key's channels.  Before the norm the read-out of those queries is that token's value,
  so after the norm it is the value's direction: a state lost at a cut, or a decay on the wrong rows, gives noise."""
  g = torch.Generator().manual_seed(3)
  H, D, Dv, T, eps = 2, 32, 16, 760, 1e-6
  r = lambda *s: torch.randn(s, generator=g)
  k = 0.02 * r(T, H, D)
  k[:, :, :4] = 0                                       # the channels of the far key: no other token writes there
  k[5] = 0
  k[5, :, :4] = 2.0
  q = 0.02 * r(T, H, D)
  q[700:, :, :4] = 8.0                                  # the last sixty tokens ask for it
  v, gate = r(T, H * Dv), r(T, H * Dv)
  q, k, v, gate = (x.reshape(T, -1).to(DT[dtype]) for x in (q, k, v, gate))
  if channel:
    logits = r(T, H * D)
    logits.view(T, H, D)[:, :, :4] = 30.0               # sigmoid(30) is 1 in float32
    alpha = torch.exp(torch.nn.functional.logsigmoid(logits) / 4.0).view(T, H, D)
    kw = dict(decay_logits=logits, tau=4.0)
  else:
    alpha = torch.tensor([1.0, 1.0])[None, :, None].expand(T, H, D)
    kw = dict(head_decay=torch.ones(2, dtype=torch.float32, device=DEV))
  want = plain_linear_attention(q.float().view(T, H, D), k.float().view(T, H, D), v.float().view(T, H, Dv), gate, alpha, eps)
  if channel:      # the far value is what comes out
    far = plain.rms_unit(v[5].float().view(H, Dv), eps) * plain.silu(gate[750].float().view(H, Dv))
    assert float((want[750] - far.reshape(-1)).abs().max()) < 0.05
  for cuts in ((T,), (6, 694) + (1,) * 60, (4, 2, 300, 394, 58, 2), (700, 2, 2, 56)):
    got, _ = run_linear_attention(cuts, dtype, q, k, v, gate, H, D, Dv, eps, **kw)
    assert float((got[700:] - want[700:]).abs().max()) <= 2 * tol(dtype), f"cut into {cuts[:6]}"
    assert float((got - want).abs().max()) <= (2 * tol(dtype) if dtype == "float32" else 0.25), f"cut into {cuts[:6]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,D,Dv,channel", [(2, 24, 40, True), (1, 128, 64, True), (3, 64, 32, False)])
def test_linear_attention_of_long_portions(dtype, H, D, Dv, channel):
  """Portions of hundreds of tokens: in bfloat16 a request's tokens run in stretches side by side, each from a zero
  state, and are chained afterwards by the products of their decays; the result is the recurrence's, and the state
  left behind lets the request go on token by token."""
  g = torch.Generator().manual_seed(D + Dv)
  T, eps = 1300, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  q, k, v, gate = (r(T, H * n).to(DT[dtype]) for n in (D, D, Dv, Dv))
  if channel:
    logits, bias = r(T, H * D), 3.0 + r(H * D)
    alpha = torch.exp(torch.nn.functional.logsigmoid(logits + bias) / 8.0).view(T, H, D)
    kw = dict(decay_logits=logits, decay_bias=bias.to(DEV), tau=8.0)
  else:
    decay = [0.9, 0.999, 0.97][:H]
    alpha = torch.tensor(decay)[None, :, None].expand(T, H, D)
    kw = dict(head_decay=torch.tensor(decay, dtype=torch.float32, device=DEV))
  qf, kf, vf = q.float().view(T, H, D) * D ** -0.5, k.float().view(T, H, D), v.float().view(T, H, Dv)
  want = plain_linear_attention(qf, kf, vf, gate, alpha, eps)
  last = torch.zeros(H, D, Dv, dtype=torch.float64)
  for t in range(T):
    last = alpha[t].double()[:, :, None] * last + kf[t].double()[:, :, None] * vf[t].double()[:, None, :]
  for cuts in ((600, 2, 690, 1, 1, 1, 1, 1, 1, 1, 1), (1290,) + (1,) * 10, (520, 780)):
    got, state = run_linear_attention(cuts, dtype, q, k, v, gate, H, D, Dv, eps, q_scale=D ** -0.5, **kw)
    assert float((got - want).abs().max()) <= 2 * tol(dtype), f"cut into {cuts[:4]}"
    assert float((state.double() - last).abs().max()) <= 2e-3 * max(1.0, float(last.abs().max()))


def test_items_of_a_step_keep_to_their_own_states():
  """Three requests in one step - a long portion, a single token, a portion of two - against each alone, to the bit."""
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(8)
  H, D, Dv, eps = 2, 24, 16, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  lens, slots = (37, 1, 2), (3, 0, 1)
  T = sum(lens)
  q, k, v, gate, logits = (r(T, H * n).to(DEV) for n in (D, D, Dv, Dv, D))
  start = torch.randn((4, H * D * Dv), generator=g).to(DEV)           # every request is in the middle of its text
  together, out = start.clone(), torch.zeros((T, H * Dv), device=DEV)
  ops.linear_attention(out, q, k, v, gate, together, step_ctx([(n, 50, s) for n, s in zip(lens, slots)]), H, D, Dv, eps, decay_logits=logits, tau=2.0)
  row = 0
  for n, s in zip(lens, slots):
    alone, o = start.clone(), torch.zeros((n, H * Dv), device=DEV)
    sl = slice(row, row + n)
    ops.linear_attention(o, q[sl], k[sl], v[sl], gate[sl], alone, step_ctx([(n, 50, s)]), H, D, Dv, eps, decay_logits=logits[sl], tau=2.0)
    if DEV != "cpu":
      assert torch.equal(o, out[sl]) and torch.equal(alone[s], together[s])
    else:
      assert torch.allclose(o, out[sl], atol=1e-5) and torch.allclose(alone[s], together[s], atol=1e-5)
    row += n
  assert torch.equal(together[2], start[2])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,W", [(1, 64), (2, 96), (3, 40), (4, 192), (5, 1000)])
def test_streams_are_mixed_all_at_once_and_read_through_their_weights(dtype, S, W):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(S * W)
  T, eps = 13, 1e-5
  r = lambda *s: torch.randn(s, generator=g)
  xs, y = r(S, T, W), r(T, W).to(DT[dtype])
  Wt = {"in": r(S), "out": r(S), "mix": torch.eye(S) + 0.5 * r(S, S)}
  nw = 1 + 0.2 * r(W)
  new = plain.hyper_sublayer(xs, Wt, "", lambda u: y.float())
  rows_of = lambda x: x.permute(1, 0, 2).reshape(T, S * W).clone()
  dev = lambda t: t.to(DEV)
  # the update, then the next sublayer's input through its own weights and norm
  streams, res = dev(rows_of(xs)).contiguous(), torch.zeros((T, W), dtype=DT[dtype], device=DEV)
  in2 = r(S)
  ops.hyper_connection(res, streams, dev(y), dev(Wt["mix"]), dev(Wt["out"]), dev(in2), dev(nw), eps)
  assert float((streams.cpu() - rows_of(new)).abs().max()) <= 1e-5
  want = plain.norm_plain(torch.einsum("s,stw->tw", in2, new), nw, eps)
  assert float((res.float().cpu() - want).abs().max()) <= tol(dtype)
  # no update: the first sublayer's input from the streams as they are
  res1 = torch.zeros((T, W), dtype=DT[dtype], device=DEV)
  before = streams.clone()
  ops.hyper_connection(res1, streams, None, None, None, dev(in2), dev(nw), eps)
  assert torch.equal(streams, before) and float((res1.float() - res.float()).abs().max()) <= tol(dtype)
  # chosen rows, not written back, read as the plain sum without a norm: what the model's last norm takes
  streams = dev(rows_of(xs)).contiguous()
  pick = torch.tensor([11, 2, 5], dtype=torch.int32)
  total = torch.zeros((3, W), dtype=torch.float32, device=DEV)
  ops.hyper_connection(total, streams, dev(y), dev(Wt["mix"]), dev(Wt["out"]), None, None, eps, rows=dev(pick), write_back=False)
  assert torch.equal(streams.cpu(), rows_of(xs))
  assert float((total.cpu() - new.sum(0)[pick.long()]).abs().max()) <= 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_small_elementwise_kernels(dtype):
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(1)
  x, y = torch.randn((7, 333), generator=g).to(DT[dtype]), torch.randn((7, 333), generator=g).to(DT[dtype])
  out = torch.zeros((7, 333), dtype=DT[dtype], device=DEV)
  ops.relu_squared(out, x.to(DEV))
  assert torch.equal(out.cpu(), (torch.relu(x.float()) ** 2).to(DT[dtype]))
  ops.scaled_pair_sum(out, x.to(DEV), y.to(DEV), 0.7, 1.3)
  assert float((out.float().cpu() - (0.7 * x.float() + 1.3 * y.float())).abs().max()) <= (1e-6 if dtype == "float32" else 2e-2)
  table = torch.randn((50, 24), generator=g).to(DT[dtype])
  ids = torch.tensor([3, 49, 0, 3], dtype=torch.int32)
  rows = torch.zeros((4, 72), dtype=torch.float32, device=DEV)
  ops.embedding(rows, table.to(DEV), ids.to(DEV), 1.0, 3)
  assert torch.equal(rows.cpu(), table[ids.long()].float().repeat(1, 3))


@pytest.mark.parametrize("M,N,K,force_tc", [(1, 72, 64, False), (8, 520, 192, False), (16, 2056, 256, False), (40, 136, 96, False),
                                            (300, 264, 128, True), (1800, 520, 320, False)])
def test_up_product_with_the_squared_relu_in_its_epilogue(M, N, K, force_tc, monkeypatch):
  """Few rows (the mma.sync kernel), many rows (the tcgen05 kernel) and what lies between (product, then activation) give
  max(bfloat16(x w^T), 0)^2; a fused kernel gives bit for bit what the same product followed by the activation kernel gives."""
  from miniinfer_b200.engine.context import Workspace
  from miniinfer_b200.kernels import ops
  g = torch.Generator().manual_seed(M + N)
  x = torch.randn((M, K), generator=g).to(torch.bfloat16)
  w = (torch.randn((N, K), generator=g) / K ** 0.5).to(torch.bfloat16)
  ws = Workspace(torch.device(DEV))
  out = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
  ops.linear_relu_squared(out, x.to(DEV), w.to(DEV), ws, force_tc=force_tc)
  prod = x.float() @ w.float().t()
  want = torch.relu(prod.to(torch.bfloat16).float()) ** 2
  # a product within a rounding step of a bfloat16 boundary may round either way: two steps of the squared value
  assert float(((out.float().cpu() - want).abs() / (want.abs() + 0.05)).max()) <= 2.5e-2
  assert float(out.float().min()) >= 0.0
  # the same product kernel, unfused
  two = torch.zeros_like(out)
  if M <= 16:
    ops.linear(two, x.to(DEV), w.to(DEV))
  elif force_tc or M >= 1792:
    ops.linear_tc(two, x.to(DEV), w.to(DEV), ws)
  else:
    monkeypatch.setenv("MINIINFER_B200_RELU2_FUSED", "0")
    ops.linear_relu_squared(two, x.to(DEV), w.to(DEV), ws)
    assert torch.equal(two, out)
    return
  ops.relu_squared(two, two)
  assert torch.equal(two, out)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,D,Dv,rot_dims", [(4, 1, 24, 16, 16), (2, 2, 16, 32, 8), (6, 3, 32, 32, 32), (2, 1, 128, 64, 32)])
def test_biases_norm_over_the_whole_projection_and_rotation(dtype, H, G, D, Dv, rot_dims):
  """Biases are added before the norm, the root mean square runs over all heads of a projection at once with a weight for
  every one of its values, the rotation comes last; the values get their bias and nothing else."""
  from miniinfer_b200.kernels import ops
  from miniinfer_b200.parts import BandScaledRotaryEncoding
  g = torch.Generator().manual_seed(H * D + rot_dims)
  T, page, eps = 11, 8, 1e-5
  hdp = -(-max(D, Dv) // 16) * 16
  scaling = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}
  rot = {"dims": rot_dims, "base": 10000.0, "scaling": scaling}
  pe = BandScaledRotaryEncoding("rot", rot_dims, 10000.0, 4096, scaling=scaling)
  pe.prepare(DEV, 128)
  nq, nk, nv = H * D, G * D, G * Dv
  proj = torch.randn((T, nq + nk + nv + H * Dv), generator=g).to(DT[dtype])
  # one head far larger than the others: a norm taken head by head would give something else altogether
  proj[:, :D] *= 6.0
  bias = torch.randn((nq + nk + nv,), generator=g)
  qw, kw = 1 + 0.2 * torch.randn((nq,), generator=g), 1 + 0.2 * torch.randn((nk,), generator=g)
  pos = torch.arange(50, 50 + T)
  x = proj.float()[:, :nq + nk + nv] + bias
  q = plain.rotate_half(plain.norm_plain(x[:, :nq], qw, eps).view(T, H, D), pos, rot)
  k = plain.rotate_half(plain.norm_plain(x[:, nq:nq + nk], kw, eps).view(T, G, D), pos, rot)
  v = x[:, nq + nk:].view(T, G, Dv)
  kv = torch.zeros((8, 2, G, page, hdp), dtype=DT[dtype], device=DEV)
  slots = torch.tensor([3 * page + 5 - j if j < 6 else 5 * page + j - 6 for j in range(T)], dtype=torch.int32, device=DEV)
  q_out = torch.full((T, H * hdp), 3.0, dtype=DT[dtype], device=DEV)
  ops.qkv_norm_mix_store(proj.to(DEV), 0, nq, nq + nk, q_out, H, G, D, Dv, eps, True, qw.to(DEV), kw.to(DEV), None, None, 0, slots, kv,
                         rope=pe.rotary_table(), positions=pos.to(torch.int32).to(DEV), interleaved=False, bias=bias.to(DEV), norm_whole=True)
  qo = q_out.float().cpu().view(T, H, hdp)
  assert float((qo[..., :D] - q).abs().max()) <= tol(dtype) * 2 and (D == hdp or float(qo[..., D:].abs().max()) == 0)
  for j in range(T):
    s = int(slots[j])
    assert float((kv[s // page, 0, :, s % page, :D].float().cpu() - k[j]).abs().max()) <= tol(dtype) * 2
    assert float((kv[s // page, 1, :, s % page, :Dv].float().cpu() - v[j]).abs().max()) <= tol(dtype) * 2
