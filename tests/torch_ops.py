"""Plain PyTorch statements of the engine's device operations, one for each function of
``miniinfer_b200.kernels.ops`` and with the same arguments.

Two uses: (1) on the GPU, each CUDA kernel is compared with its statement here; (2) on the CPU,
``install(monkeypatch)`` puts these in place of the kernels so that the host-side logic of the
engine (cache manager, step metadata, scheduler, replay) can be tested without a device.  They are
test code only; the package itself has no implementation other than its CUDA kernels.

All arithmetic is float32 (float64 where noted) on whatever device the tensors are on.
"""

from __future__ import annotations

import math
from typing import Optional

import torch


def embedding(out, table, ids, scale=1.0, copies=1):
  out.copy_((table[ids.long()].float() * scale).repeat(1, copies))


def add_layernorm(out, resid, delta, delta2, weight, bias, eps, rows=None, write_back=True):
  idx = rows.long() if rows is not None else None
  x = resid if idx is None else resid[idx]
  ds = [d for d in (delta, delta2) if d is not None]
  if ds:
    add = ds[0].float() if len(ds) == 1 else ds[0].float() + ds[1].float()
    x = x + (add if idx is None else add[idx])
    if write_back:
      if idx is None:
        resid.copy_(x)
      else:
        resid[idx] = x
  mu = x.mean(-1, keepdim=True)
  var = ((x - mu) ** 2).mean(-1, keepdim=True)
  out.copy_(((x - mu) / torch.sqrt(var + eps) * weight + bias).to(out.dtype))


def add_rmsnorm(out, resid, delta, weight, eps, rows=None, write_back=True):
  idx = rows.long() if rows is not None else None
  x = resid if idx is None else resid[idx]
  if delta is not None:
    x = x + (delta if idx is None else delta[idx]).float()
    if write_back:
      if idx is None:
        resid.copy_(x)
      else:
        resid[idx] = x
  var = x.pow(2).mean(-1, keepdim=True)
  out.copy_((weight * (x * torch.rsqrt(var + eps))).to(out.dtype))


def linear(out, x, w, force_skinny=False):
  out.copy_((x.float() @ w.float().t()).to(out.dtype))


def _rms(resid, weight, eps):
  x = resid.float()
  return (weight * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))).to(torch.bfloat16)


def linear_normed(out, resid, norm_weight, eps, w):
  linear(out, _rms(resid, norm_weight, eps), w)


def linear_swiglu_normed(out, resid, norm_weight, eps, w):
  linear_swiglu(out, _rms(resid, norm_weight, eps), w, None)


def linear_add(resid, x, w):
  resid.add_((x.float() @ w.float().t()).to(torch.bfloat16).float())


def qk_norm_rope_store(qkv, q_weight, k_weight, cos_sin, positions, slot_mapping, kv_layer,
                       num_heads, num_kv_heads, head_dim, eps):
  T = qkv.shape[0]
  nh, nkv, hd = num_heads, num_kv_heads, head_dim
  x = qkv.float().view(T, nh + 2 * nkv, hd)
  q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

  def norm(t, w):
    if w is None:
      return t
    return w * (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps))

  def rope(t):
    if cos_sin is None:
      return t
    rot = cos_sin.shape[1]
    cs = cos_sin[positions.long()]
    c, s = cs[:, None, :rot // 2], cs[:, None, rot // 2:]
    t1, t2, rest = t[..., :rot // 2], t[..., rot // 2:rot], t[..., rot:]
    return torch.cat((t1 * c - t2 * s, t2 * c + t1 * s, rest), dim=-1)

  q = rope(norm(q, q_weight))
  k = rope(norm(k, k_weight))
  res = torch.cat((q, k, v), dim=1).reshape(T, -1).to(qkv.dtype)
  qkv.copy_(res)
  if slot_mapping is not None and kv_layer is not None:
    P = kv_layer.shape[3]
    r = res.view(T, nh + 2 * nkv, hd)
    slot = slot_mapping.long()
    ok = slot >= 0
    page, off = (slot // P)[ok], (slot % P)[ok]
    kv_layer[page, 0, :, off, :] = r[ok, nh:nh + nkv]
    kv_layer[page, 1, :, off, :] = r[ok, nh + nkv:]


def qkv_norm_mix_store(proj, q_off, k_off, v_off, q_out, num_heads, num_kv_heads, dim, vdim, eps, normalise=True,
                       q_weight=None, k_weight=None, mix=None, v_other=None, v_mode=0, slot_mapping=None, kv_layer=None,
                       rope=None, positions=None, interleaved=False, bias=None, norm_whole=False):
  T = proj.shape[0]
  H, G = num_heads, num_kv_heads
  hdp = q_out.shape[1] // H
  x = proj.float()
  if bias is not None:
    x = x.clone()
    x[:, :bias.shape[0]] += bias
  q = x[:, q_off:q_off + H * dim].reshape(T, H, dim)
  k = x[:, k_off:k_off + G * dim].reshape(T, G, dim)
  v = x[:, v_off:v_off + G * vdim].reshape(T, G, vdim)
  if normalise:
    over = (-2, -1) if norm_whole else -1
    q = q / torch.sqrt(q.pow(2).mean(over, keepdim=True) + eps)
    k = k / torch.sqrt(k.pow(2).mean(over, keepdim=True) + eps)
  if q_weight is not None:
    q = q * (q_weight.view(H, dim) if norm_whole else q_weight)
  if k_weight is not None:
    k = k * (k_weight.view(G, dim) if norm_whole else k_weight)
  if rope is not None:
    q, k = _rotate(q, rope, positions, interleaved), _rotate(k, rope, positions, interleaved)
  if v_mode == 1:
    v_other.copy_(v.reshape(T, G * vdim).to(v_other.dtype))
  elif v_mode == 2:
    lam = mix.float()
    v = (1 - lam) * v + lam * v_other.float().reshape(T, G, vdim)
  qp = torch.zeros((T, H, hdp), dtype=torch.float32, device=proj.device)
  qp[..., :dim] = q
  q_out.copy_(qp.reshape(T, H * hdp).to(q_out.dtype))
  if slot_mapping is not None and kv_layer is not None:
    P = kv_layer.shape[3]
    slot = slot_mapping.long()
    page, off = slot // P, slot % P
    kp = torch.zeros((T, G, hdp), dtype=torch.float32, device=proj.device)
    vp = torch.zeros((T, G, hdp), dtype=torch.float32, device=proj.device)
    kp[..., :dim] = k
    vp[..., :vdim] = v
    kv_layer[page, 0, :, off, :] = kp.to(kv_layer.dtype)
    kv_layer[page, 1, :, off, :] = vp.to(kv_layer.dtype)


def _rotate(t, table, positions, interleaved):
  """t [T, heads, size]: the first table.shape[1] values of every head rotated by the angles of the token's position."""
  rot = table.shape[1]
  cs = table[positions.long()]
  c, s = cs[:, None, :rot // 2], cs[:, None, rot // 2:]
  out = t.clone()
  if interleaved:
    u, v = t[..., 0:rot:2], t[..., 1:rot:2]
    out[..., 0:rot:2], out[..., 1:rot:2] = u * c - v * s, v * c + u * s
  else:
    u, v = t[..., :rot // 2], t[..., rot // 2:rot]
    out[..., :rot // 2], out[..., rot // 2:rot] = u * c - v * s, v * c + u * s
  return out


def _glu(g, u, glu, limit):
  if glu == "clamped":
    g, u = torch.clamp(g, max=limit), torch.clamp(u, -limit, limit)
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)
  return g * torch.sigmoid(g) * u


def routed_experts(out, x, router, correction, gate_up, down, top, workspace, weights="sigmoid_share", glu="silu", limit=0.0,
                   shared=None, shared_gated=False):
  T, H = x.shape
  E, ff = down.shape[0], down.shape[2]
  z = x.float() @ router.float().t()
  if weights == "softmax_chosen":
    idx = torch.topk(z[:, :E], top, dim=-1).indices
    w = torch.softmax(torch.gather(z, 1, idx), dim=-1)
  else:
    s = torch.sigmoid(z[:, :E])
    idx = torch.topk(s + correction, top, dim=-1).indices
    w = torch.gather(s, 1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20)
  res = torch.zeros((T, H), dtype=torch.float32, device=x.device)
  for e in range(E):
    g = x.float() @ gate_up[e, :ff].float().t()
    u = x.float() @ gate_up[e, ff:].float().t()
    act = _glu(g, u, glu, limit).to(x.dtype).float()
    y = act @ down[e].float().t()
    res += (w * (idx == e)).sum(-1, keepdim=True) * y
  if shared is not None:
    res += shared.float() * (torch.sigmoid(z[:, E:E + 1]) if shared_gated else 1.0)
  out.copy_(res.to(out.dtype))


def glu_mul(out, gate_up, glu="silu", limit=0.0):
  I = out.shape[1]
  out.copy_(_glu(gate_up[:, :I].float(), gate_up[:, I:].float(), glu, limit).to(out.dtype))


def linear_glu(out, x, w, workspace, glu="silu", limit=0.0):
  gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype)
  linear(gu, x, w)
  glu_mul(out, gu, glu, limit)


def token_shift(out, resid, shift, state, ctx):
  if shift is None:
    out.copy_(resid.to(out.dtype))
    return
  W = resid.shape[1]
  for row0, n, slot in _items(ctx):
    x = resid[row0:row0 + n]
    before = torch.cat((state[slot, :W][None], x[:-1]), dim=0)
    out[row0:row0 + n] = (x + (before - x) * shift).to(out.dtype)


def norm_scaled_add(resid, y, weight, eps, mult, ctx, copy=None, keep=None):
  W = resid.shape[1]
  if keep is not None:
    for row0, n, slot in _items(ctx):
      keep[slot, :W] = resid[row0 + n - 1]
  v = y.float()
  resid += mult * weight * (v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps))
  if copy is not None:
    copy.copy_(resid.to(copy.dtype))


def rglru_recurrence(out, u, gates, y, r_bias, i_bias, y_bias, lam, state, ctx, blocks, workspace=None):
  T, C = u.shape
  P = C // blocks
  g = gates.transpose(0, 1) if gates.dim() == 3 else gates.view(T, blocks, 2 * P)
  r = torch.sigmoid(g[:, :, :P].reshape(T, C) + r_bias)
  i = torch.sigmoid(g[:, :, P:].reshape(T, C) + i_bias)
  log_a = -8.0 * r * torch.nn.functional.softplus(lam)
  a = torch.exp(log_a)
  b = torch.sqrt(-torch.expm1(2.0 * log_a)) * i * u.float()
  yy = y.float() + (y_bias if y_bias is not None else 0.0)
  gate = 0.5 * yy * (1.0 + torch.tanh(0.7978845608028654 * (yy + 0.044715 * yy ** 3)))
  _diagonal(out, a, b, gate, state, ctx, C)


def mingru_recurrence(out, proj, z_bias, x_bias, state, ctx, workspace=None):
  C = out.shape[1]
  zl = proj[:, :C].float() + (z_bias if z_bias is not None else 0.0)
  x = proj[:, C:2 * C].float() + (x_bias if x_bias is not None else 0.0)
  g = proj[:, 2 * C:].float()
  z = torch.sigmoid(zl)
  _diagonal(out, 1.0 - z, z * torch.where(x >= 0, x + 0.5, torch.sigmoid(x)), g * torch.sigmoid(g), state, ctx, C)


def _diagonal(out, a, b, gate, state, ctx, C):
  for row0, n, slot in _items(ctx):
    S = state[slot, :C].clone()
    for t in range(row0, row0 + n):
      S = a[t] * S + b[t]
      out[t] = (S * gate[t]).to(out.dtype)
    state[slot, :C] = S


def attention(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale, window,
              force_generic=False, sink=None, gate=None, gate_offset=0, out_hd=None, keep_first=0, softcap=0.0, score_bias=None):
  if sink is not None or gate is not None or (out_hd is not None and out_hd != head_dim) or keep_first or softcap or score_bias is not None:
    return _attention_with_options(out, qkv, kv_layer, block_table, batch, num_heads, num_kv_heads, head_dim, scale,
                                   window, sink, gate, gate_offset, out_hd if out_hd is not None else head_dim, keep_first,
                                   softcap, score_bias)
  T = qkv.shape[0]
  nh, nkv, hd = num_heads, num_kv_heads, head_dim
  P = kv_layer.shape[3]
  g = nh // nkv
  q = qkv.float().view(T, -1, hd)[:, :nh]
  pos = batch.positions.tolist()
  item = batch.token_item.tolist()
  slots = batch.seq_slot.tolist()
  res = torch.zeros((T, nh, hd), dtype=torch.float32, device=qkv.device)
  for t in range(T):
    p = pos[t]
    lo = max(0, p - window + 1) if window else 0
    js = torch.arange(lo, p + 1, device=qkv.device)
    pages = block_table[slots[item[t]]].long()[js // P]
    k = kv_layer[pages, 0, :, js % P, :].float()          # [n, nkv, hd]
    v = kv_layer[pages, 1, :, js % P, :].float()
    k = k.repeat_interleave(g, dim=1)                     # [n, nh, hd]
    v = v.repeat_interleave(g, dim=1)
    s = torch.einsum("hd,nhd->hn", q[t], k) * scale
    pr = torch.softmax(s, dim=-1)
    res[t] = torch.einsum("hn,nhd->hd", pr, v)
  out.copy_(res.reshape(T, nh * hd).to(out.dtype))


def _attention_with_options(out, qkv, kv_layer, block_table, batch, nh, nkv, hd, scale, window, sink, gate, gate_offset, ohd,
                            keep_first=0, softcap=0.0, score_bias=None):
  T = qkv.shape[0]
  P = kv_layer.shape[3]
  g = nh // nkv
  q = qkv.float().view(T, -1, hd)[:, :nh]
  pos, item, slots = batch.positions.tolist(), batch.token_item.tolist(), batch.seq_slot.tolist()
  res = torch.zeros((T, nh, ohd), dtype=torch.float32, device=qkv.device)
  for t in range(T):
    p = pos[t]
    lo = max(0, p - window + 1) if window else 0
    js = torch.arange(lo, p + 1, device=qkv.device)
    if window and keep_first:
      js = torch.cat((torch.arange(0, min(keep_first, lo), device=qkv.device), js))
    pages = block_table[slots[item[t]]].long()[js // P]
    k = kv_layer[pages, 0, :, js % P, :].float().repeat_interleave(g, dim=1)
    v = kv_layer[pages, 1, :, js % P, :].float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,nhd->hn", q[t], k) * scale
    if softcap:
      s = softcap * torch.tanh(s / softcap)
    if score_bias is not None:
      res[t] = torch.einsum("hn,nhd->hd", torch.sigmoid(s + score_bias[:, None]), v)[:, :ohd]
      continue
    if sink is not None:
      s = torch.cat((s, sink.float()[:, None]), dim=1)
    pr = torch.softmax(s, dim=-1)[:, :js.numel()]
    res[t] = torch.einsum("hn,nhd->hd", pr, v)[:, :ohd]
  res = res.reshape(T, nh * ohd)
  if gate is not None:
    res = res * torch.sigmoid(gate.float()[:, gate_offset:gate_offset + nh * ohd])
  out.copy_(res.to(out.dtype))


def add_rmsnorm_pair(out1, out2, resid, delta, delta2, w1, w2, eps, rows=None, write_back=True):
  idx = rows.long() if rows is not None else None
  x = resid if idx is None else resid[idx]
  ds = [d for d in (delta, delta2) if d is not None]
  if ds:
    add = ds[0].float() if len(ds) == 1 else ds[0].float() + ds[1].float()
    x = x + (add if idx is None else add[idx])
    if write_back:
      if idx is None:
        resid.copy_(x)
      else:
        resid[idx] = x
  n = x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)
  out1.copy_((w1 * n).to(out1.dtype))
  if out2 is not None:
    out2.copy_((w2 * n).to(out2.dtype))


def rms_pair_sum(out, a, b, w1, w2, eps, scale):
  def unit(t):
    t = t.float()
    return t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps)
  out.copy_((scale * (w1 * unit(a) + w2 * unit(b))).to(out.dtype))


def linear_batched(out, x, w, bias=None, softplus=False, row_gate=None):
  y = torch.einsum("mbk,bnk->mbn", x.float(), w.float())
  if bias is not None:
    y = y + bias
  if softplus:
    y = torch.nn.functional.softplus(y)
  if row_gate is not None:
    y = y * torch.sigmoid(row_gate.float()[:, :x.shape[1], None])
  out.copy_(y.to(out.dtype))


def linear_parts(out, x, w):
  B, N, K = w.shape
  out.copy_(torch.einsum("mbk,bnk->bmn", x.float().view(x.shape[0], B, K), w.float()).to(out.dtype))


def _items(ctx):
  return list(zip(ctx.q_start.tolist(), ctx.q_len.tolist(), ctx.seq_slot.tolist()))


def causal_conv(out, x, weight, bias, state, ctx, silu=True, in_bias=None):
  C, taps = weight.shape
  S = taps - 1
  for row0, n, slot in _items(ctx):
    old = state[slot, :S * C].view(S, C) if S else x.new_zeros((0, C), dtype=torch.float32)
    seq = torch.cat((old.float(), x[row0:row0 + n].float() + (in_bias if in_bias is not None else 0.0)), dim=0)
    y = sum(seq[k:k + n] * weight[:, k] for k in range(taps))
    if bias is not None:
      y = y + bias
    if silu:
      y = y * torch.sigmoid(y)
    out[row0:row0 + n] = y.to(out.dtype)
    if S:
      state[slot, :S * C] = seq[seq.shape[0] - S:].reshape(-1)


def selective_scan(y, u, dt_in, bc, b_off, c_off, z, dt_bias, A_log, D, state, ctx, workspace=None):
  inner, N = A_log.shape
  A = -torch.exp(A_log.float())
  for row0, n, slot in _items(ctx):
    S = state[slot, :inner * N].view(inner, N).clone()
    for t in range(row0, row0 + n):
      dt = torch.nn.functional.softplus(dt_in[t].float() + dt_bias)
      ut = u[t].float()
      S = torch.exp(dt[:, None] * A) * S + (dt * ut)[:, None] * bc[t, b_off:b_off + N].float()[None, :]
      zt = z[t].float()
      y[t] = ((S @ bc[t, c_off:c_off + N].float() + D * ut) * (zt * torch.sigmoid(zt))).to(y.dtype)
    state[slot, :inner * N] = S.reshape(-1)


def gated_delta(out, q, k, v, a, b, gate, dt_bias, A_log, norm_w, eps, state, ctx, heads, kv_heads, dim, vdim, workspace=None):
  H, G, D, Dv = heads, kv_heads, dim, vdim
  for row0, n, slot in _items(ctx):
    S = state[slot, :H * D * Dv].view(H, D, Dv).clone()
    for t in range(row0, row0 + n):
      qt, kt = q[t].float().view(G, D), k[t].float().view(G, D)
      qt = qt / torch.sqrt(qt.pow(2).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
      kt = kt / torch.sqrt(kt.pow(2).sum(-1, keepdim=True) + 1e-6)
      qt, kt = qt.repeat_interleave(H // G, dim=0), kt.repeat_interleave(H // G, dim=0)        # [H, D]
      g = torch.exp(-torch.exp(A_log.float())[:, None] * torch.nn.functional.softplus(a[t].float().view(H, D) + dt_bias.view(H, D)))
      beta = torch.sigmoid(b[t].float())                                                       # [H]
      S = g[:, :, None] * S
      u = beta[:, None] * (v[t].float().view(H, Dv) - torch.einsum("hdv,hd->hv", S, kt))
      S = S + kt[:, :, None] * u[:, None, :]
      o = torch.einsum("hdv,hd->hv", S, qt)
      o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * norm_w * torch.sigmoid(gate[t].float().view(H, Dv))
      out[t] = o.reshape(-1).to(out.dtype)
    state[slot, :H * D * Dv] = S.reshape(-1)


def linear_attention(out, q, k, v, gate, state, ctx, heads, dim, vdim, eps, decay_logits=None, decay_bias=None, tau=1.0,
                     head_decay=None, rope=None, q_scale=1.0, k_scale=1.0, norm_weight=None, gate_silu=True, workspace=None):
  H, D, Dv = heads, dim, vdim
  T = v.shape[0]
  qf, kf = q.float().reshape(T, H, D), k.float().reshape(T, H, D)
  if rope is not None:
    qf, kf = _rotate(qf, rope, ctx.positions, False), _rotate(kf, rope, ctx.positions, False)
  qf, kf = qf * q_scale, kf * k_scale
  if decay_logits is not None:
    z = decay_logits.float() + (decay_bias if decay_bias is not None else 0.0)
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, H, D)
  else:
    alpha = head_decay.float()[None, :, None].expand(T, H, D)
  for row0, n, slot in _items(ctx):
    S = state[slot, :H * D * Dv].view(H, D, Dv).clone()
    for t in range(row0, row0 + n):
      S = alpha[t][:, :, None] * S + kf[t][:, :, None] * v[t].float().view(H, 1, Dv)
      o = torch.einsum("hdv,hd->hv", S, qf[t])
      o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps)
      if norm_weight is not None:
        o = o * norm_weight
      g = gate[t].float().view(H, Dv)
      out[t] = (o * (g * torch.sigmoid(g) if gate_silu else torch.sigmoid(g))).reshape(-1).to(out.dtype)
    state[slot, :H * D * Dv] = S.reshape(-1)


def hyper_connection(res, streams, y, mix, out_w, in_w, norm_weight, eps, rows=None, write_back=True):
  W = res.shape[1]
  S = streams.shape[1] // W
  idx = rows.long() if rows is not None else None
  x = (streams if idx is None else streams[idx]).view(-1, S, W)
  if y is not None:
    yy = (y if idx is None else y[idx]).float()
    x = torch.einsum("st,nsw->ntw", mix, x) + out_w[None, :, None] * yy[:, None, :]
    if write_back:
      if idx is None:
        streams.copy_(x.reshape(-1, S * W))
      else:
        streams[idx] = x.reshape(-1, S * W)
  u = x.sum(1) if in_w is None else torch.einsum("s,nsw->nw", in_w, x)
  if norm_weight is not None:
    u = norm_weight * (u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + eps))
  res.copy_(u.to(res.dtype))


def relu_squared(out, x):
  out.copy_((torch.relu(x.float()) ** 2).to(out.dtype))


def linear_relu_squared(out, x, w, workspace, force_tc=False):
  linear(out, x, w)
  relu_squared(out, out)


def scaled_pair_sum(out, a, b, scale_a, scale_b):
  out.copy_((scale_a * a.float() + scale_b * b.float()).to(out.dtype))


def latent_down(down, q_off, kv_off, q_rank, kv_rank, rot_dim, q_weight, kv_weight, eps, cq_out, rope, positions, interleaved,
                slot_mapping, kv_layer):
  T = down.shape[0]
  x = down.float()

  def unit(t):
    return t / torch.sqrt(t.pow(2).mean(-1, keepdim=True) + eps)

  cq_out.copy_((q_weight * unit(x[:, q_off:q_off + q_rank])).to(cq_out.dtype))
  if slot_mapping is None or kv_layer is None:
    return
  c = kv_weight * unit(x[:, kv_off:kv_off + kv_rank])
  kr = _rotate(x[:, None, kv_off + kv_rank:kv_off + kv_rank + rot_dim], rope, positions, interleaved)[:, 0]
  P, hdp = kv_layer.shape[3], kv_layer.shape[4]
  krow = torch.zeros((T, hdp), dtype=torch.float32, device=down.device)
  vrow = torch.zeros((T, hdp), dtype=torch.float32, device=down.device)
  krow[:, :kv_rank], krow[:, kv_rank:kv_rank + rot_dim], vrow[:, :kv_rank] = c, kr, c
  slot = slot_mapping.long()
  kv_layer[slot // P, 0, 0, slot % P, :] = krow.to(kv_layer.dtype)
  kv_layer[slot // P, 1, 0, slot % P, :] = vrow.to(kv_layer.dtype)


def latent_query(q, q_out, heads, dim, rot_dim, kv_rank, rope, positions, interleaved):
  T = q.shape[0]
  hdp = q_out.shape[1] // heads
  qr = _rotate(q.float().view(T, heads, dim + rot_dim)[:, :, dim:], rope, positions, interleaved)
  dst = q_out.view(T, heads, hdp)
  dst[:, :, kv_rank:kv_rank + rot_dim] = qr.to(q_out.dtype)
  dst[:, :, kv_rank + rot_dim:] = 0


def linear_swiglu(out, x, w, workspace, force_skinny=False, force_tc=False):
  gu = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype)
  linear(gu, x, w)
  silu_mul(out, gu)


def silu_mul(out, gate_up):
  I = out.shape[1]
  g, u = gate_up[:, :I].float(), gate_up[:, I:].float()
  out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


_M = (1 << 64) - 1


def _mix64(x: int) -> int:
  x &= _M
  x ^= x >> 30
  x = (x * 0xBF58476D1CE4E5B9) & _M
  x ^= x >> 27
  x = (x * 0x94D049BB133111EB) & _M
  x ^= x >> 31
  return x


def gumbel_scores(logits_row, temperature, top_k, top_p, seed, counter):
  """The perturbed scores whose arg-max is the sampled token (float64), -inf where filtered out."""
  V = logits_row.numel()
  z = logits_row.double().cpu() / temperature
  if top_k and 0 < top_k < V:
    kth = torch.topk(z, top_k).values[-1]
    z = torch.where(z >= kth, z, torch.full_like(z, float("-inf")))
  if top_p < 1.0:
    pr = torch.softmax(z, dim=-1)
    sp, _ = torch.sort(pr, descending=True)
    before = torch.cumsum(sp, 0) - sp
    last = int((before < top_p).nonzero().max())
    z = torch.where(pr >= sp[last], z, torch.full_like(z, float("-inf")))
  key = _mix64((seed & _M) ^ _mix64(counter + 0x9E3779B97F4A7C15))
  u = torch.tensor([((_mix64(key ^ ((i * 0xD1342543DE82EF95) & _M)) >> 41) + 0.5) / (1 << 23) for i in range(V)],
                   dtype=torch.float64)
  return z - torch.log(-torch.log(u))


def sample(out, logits, temperature, top_k, top_p, seed, counter, workspace=None):
  R = logits.shape[0]
  for r in range(R):
    t = float(temperature[r])
    if t <= 0:
      out[r] = int(torch.argmax(logits[r].float()))
    else:
      sc = gumbel_scores(logits[r], t, int(top_k[r]), float(top_p[r]), int(seed[r]), int(counter[r]))
      out[r] = int(torch.argmax(sc))


def install(monkeypatch) -> None:
  """Puts the statements above in place of the CUDA kernels (CPU tests of the host-side logic)."""
  from miniinfer_b200.kernels import ops

  for name in ("embedding", "add_rmsnorm", "add_layernorm", "linear", "linear_swiglu", "qk_norm_rope_store", "qkv_norm_mix_store",
               "attention", "routed_experts", "silu_mul", "sample", "linear_normed", "linear_swiglu_normed", "linear_add",
               "add_rmsnorm_pair", "rms_pair_sum", "linear_batched", "causal_conv", "selective_scan", "gated_delta", "latent_down",
               "latent_query", "linear_attention", "hyper_connection", "relu_squared", "linear_relu_squared", "scaled_pair_sum",
               "glu_mul", "linear_glu", "linear_parts", "token_shift", "norm_scaled_add", "rglru_recurrence", "mingru_recurrence"):
    monkeypatch.setattr(ops, name, globals()[name])
