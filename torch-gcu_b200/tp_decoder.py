"""Tensor-parallel Llama-style decoder harness (benchmark / test code, not a
reference component: the reference ships no model code, only the communication
backend that tensor parallelism is built on).

One layer: RMSNorm -> fused QKV projection (column-parallel) -> RoPE -> causal
GQA attention -> o_proj (row-parallel, all-reduce) -> residual + RMSNorm ->
gate/up projection (column-parallel) -> SwiGLU -> down projection (row-parallel,
all-reduce) -> residual. Heads and FFN columns are sharded over `tp` ranks;
activations are replicated; the KV cache shards with the KV heads.

backend "gcu": every operator runs through the registered PrivateUse1 kernels
(mm, the fused efficient ops, flash attention, add) and the all-reduce through
the registered "eccl" process group. backend "cpu": the same computation in
plain fp32 torch, used by the gloo sharding test and as the CPU baseline.
"""
import torch
import torch.nn.functional as F


def _rope_cpu(x, cos, sin, positions=None):
    B, S = x.shape[0], x.shape[1]
    if positions is None:
        positions = torch.arange(S).expand(B, S)
    c = torch.cat((cos, cos), -1)[positions][:, :, None, :]
    s = torch.cat((sin, sin), -1)[positions][:, :, None, :]
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), -1)
    return (x.float() * c + rot.float() * s).to(x.dtype)


def _rms_cpu(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def rope_tables_cpu(n, head_dim, theta=10000.0):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    fr = torch.outer(torch.arange(n, dtype=torch.float32), inv)
    return fr.cos().contiguous(), fr.sin().contiguous()


def reference_layer_cpu(x, w, hidden, heads, kv_heads, head_dim, ffn, eps=1e-6, theta=10000.0):
    """Unsharded layer in plain torch on the CPU (fp32 math on the given weights)."""
    B, S, _ = x.shape
    cos, sin = rope_tables_cpu(S, head_dim, theta)
    h = _rms_cpu(x, w["norm1"], eps)
    qkv = h.float() @ w["wqkv"].float().t()
    q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], -1)
    q = _rope_cpu(q.view(B, S, heads, head_dim), cos, sin).transpose(1, 2)
    k = _rope_cpu(k.view(B, S, kv_heads, head_dim), cos, sin).transpose(1, 2)
    v = v.view(B, S, kv_heads, head_dim).transpose(1, 2)
    g = heads // kv_heads
    att = F.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), is_causal=True)
    o = att.transpose(1, 2).reshape(B, S, heads * head_dim) @ w["wo"].float().t()
    r = x.float() + o
    h2 = _rms_cpu(r, w["norm2"], eps)
    gu = h2 @ w["wgu"].float().t()
    gate, up = gu.split(ffn, -1)
    return r + (F.silu(gate) * up) @ w["wd"].float().t()


def reference_decode_cpu(x, k_cache, v_cache, pos, w, hidden, heads, kv_heads, head_dim, ffn, eps=1e-6, theta=10000.0):
    """One decode step of the unsharded layer in plain fp32 torch on the CPU: x (n,1,hidden) new
    tokens at position `pos`, caches (n, kv_heads, T, D) whose row `pos` the step replaces.
    Returns (output (n,1,hidden), new key rows (n, kv_heads, D), new value rows)."""
    n = x.shape[0]
    cos, sin = rope_tables_cpu(k_cache.shape[2], head_dim, theta)
    positions = torch.full((n, 1), pos, dtype=torch.int64)
    h = _rms_cpu(x, w["norm1"], eps)
    qkv = h.float() @ w["wqkv"].float().t()
    q, k, v = qkv.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], -1)
    q = _rope_cpu(q.view(n, 1, heads, head_dim), cos, sin, positions).transpose(1, 2)
    k = _rope_cpu(k.view(n, 1, kv_heads, head_dim), cos, sin, positions).transpose(1, 2)
    v = v.view(n, 1, kv_heads, head_dim).transpose(1, 2)
    kc, vc = k_cache[:, :, :pos + 1].float().clone(), v_cache[:, :, :pos + 1].float().clone()
    kc[:, :, pos] = k[:, :, 0].to(k_cache.dtype).float()   # the cache holds the rows in its own dtype
    vc[:, :, pos] = v[:, :, 0].to(v_cache.dtype).float()
    g = heads // kv_heads
    att = F.scaled_dot_product_attention(q, kc.repeat_interleave(g, 1), vc.repeat_interleave(g, 1), is_causal=False)
    o = att.transpose(1, 2).reshape(n, 1, heads * head_dim) @ w["wo"].float().t()
    r = x.float() + o
    h2 = _rms_cpu(r, w["norm2"], eps)
    gu = h2 @ w["wgu"].float().t()
    gate, up = gu.split(ffn, -1)
    return r + (F.silu(gate) * up) @ w["wd"].float().t(), k[:, :, 0], v[:, :, 0]


def unfused_layer_autocast(x, p, heads, kv_heads, head_dim, eps=1e-6, theta=10000.0):
    """The decoder layer written the way a model author writes it, out of stock ATen operators only
    (pow / mean / rsqrt / mul, mm, cat, F.scaled_dot_product_attention, silu, add): no fused entry point of
    this backend is called by name. Meant to run under `torch.autocast("gcu", dtype=torch.bfloat16)` with
    fp32 parameters: the autocast policy casts the operands of every mm and of the attention to bf16 and
    keeps pow / mean / rsqrt in fp32 (reference: torch_gcu/csrc/aten/gcu_autocast_ops.cpp:28-72).
    p: wq, wk, wv, wo, wg, wu, wd, n1, n2."""
    B, S, H = x.shape

    def rms(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w

    cos_h, sin_h = rope_tables_cpu(S, head_dim, theta)
    cos = torch.cat((cos_h, cos_h), -1)[None, :, None, :].to(x.device)
    sin = torch.cat((sin_h, sin_h), -1)[None, :, None, :].to(x.device)

    def rope(t):
        half = head_dim // 2
        rot = torch.cat((-t[..., half:], t[..., :half]), -1)
        return t * cos + rot * sin

    h = rms(x, p["n1"]).view(B * S, H)
    q = rope(torch.mm(h, p["wq"].t()).view(B, S, heads, head_dim)).transpose(1, 2)
    k = rope(torch.mm(h, p["wk"].t()).view(B, S, kv_heads, head_dim)).transpose(1, 2)
    v = torch.mm(h, p["wv"].t()).view(B, S, kv_heads, head_dim).transpose(1, 2)
    att = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
    r = x + torch.mm(att.transpose(1, 2).reshape(B * S, heads * head_dim), p["wo"].t()).view(B, S, H)
    h2 = rms(r, p["n2"]).view(B * S, H)
    mlp = torch.mm(F.silu(torch.mm(h2, p["wg"].t())) * torch.mm(h2, p["wu"].t()), p["wd"].t())
    return r + mlp.view(B, S, H)


class HostExchange:
    """CPU stand-in for torch_gcu.distributed.tp_exchange.TensorParallelExchange over a gloo group: the same
    buffers, row ownership and call sequence, with the fused kernel's arithmetic written in plain torch
    (sum of the partial products, residual add, one rounding, RMSNorm, gather). It exists so that the
    sequence-parallel schedule of the exchange path runs on CPU ranks; it is not a product path."""

    def __init__(self, total_rows, hidden, dtype, group, scatter=True):
        import torch.distributed as dist
        self.group, self.scatter = group, scatter
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.total_rows, self.hidden = total_rows, hidden
        self.rows = total_rows // self.world if scatter else total_rows
        self.row0 = self.rank * self.rows if scatter else 0
        self.partial = (torch.zeros(total_rows, hidden, dtype=dtype), torch.zeros(total_rows, hidden, dtype=dtype))
        self.gathered = torch.zeros(total_rows, hidden, dtype=dtype)

    def sync(self, channel=0, signal=True, wait=True):
        pass   # the gloo collectives below are synchronous

    def reduce_norm(self, partial, residual, residual_out, weight, eps=1e-6, normalise=True):
        import torch.distributed as dist
        acc = torch.zeros(self.rows, self.hidden, dtype=torch.float32)
        if partial is not None:
            total = self.partial[partial].float().clone()
            dist.all_reduce(total, group=self.group)
            acc = total[self.row0:self.row0 + self.rows]
        if residual is not None:
            acc = acc + residual.float()
        h = acc.to(self.gathered.dtype)
        if residual_out is not None:
            residual_out.copy_(h)
        y = _rms_cpu(h, weight, eps) if normalise else h
        if self.scatter:
            parts = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(parts, y.contiguous(), group=self.group)
            self.gathered.copy_(torch.cat(parts, 0))
        else:
            self.gathered.copy_(y)


class DecoderLayer:
    def __init__(self, weights, tp, backend, hidden, heads, kv_heads, head_dim, ffn, eps=1e-6, theta=10000.0,
                 device=None):
        assert heads % tp == 0 and kv_heads % tp == 0 and ffn % tp == 0
        self.tp, self.backend, self.eps, self.theta = tp, backend, eps, theta
        self.hidden, self.head_dim = hidden, head_dim
        self.hq, self.hk, self.f = heads // tp, kv_heads // tp, ffn // tp
        self.device = device
        self.w = {k: (v.to(device) if device is not None else v) for k, v in weights.items()}
        self._tables = {}
        if backend == "gcu":
            from torch_gcu.gcu import efficient
            self.eff = efficient

    def tables(self, n):
        if n not in self._tables:
            cos, sin = rope_tables_cpu(n, self.head_dim, self.theta)
            if self.device is not None:
                cos, sin = cos.to(self.device), sin.to(self.device)
            self._tables[n] = (cos, sin)
        return self._tables[n]

    def _allreduce(self, t, group):
        if self.tp > 1:
            import torch.distributed as dist
            dist.all_reduce(t, group=group)
        return t

    # ------------------------------------------------------------- prefill --
    def attn_part(self, x, kv_out=None):
        """RMSNorm -> qkv -> RoPE -> attention -> o_proj; returns this rank's partial (B*S, hidden)."""
        B, S, H = x.shape
        hq, hk, d, w = self.hq, self.hk, self.head_dim, self.w
        cos, sin = self.tables(S)
        if self.backend != "gcu":   # plain torch, fp32 math on whatever dtype the weights have
            h = _rms_cpu(x, w["norm1"], self.eps)
            qkv = (h.float() @ w["wqkv"].float().t()).view(B, S, hq + 2 * hk, d)
            q = _rope_cpu(qkv[:, :, :hq], cos, sin).transpose(1, 2)
            k = _rope_cpu(qkv[:, :, hq:hq + hk], cos, sin).transpose(1, 2)
            v = qkv[:, :, hq + hk:].transpose(1, 2)
            g = hq // hk
            att = F.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), is_causal=True)
            return (att.transpose(1, 2).reshape(B, S, hq * d) @ w["wo"].float().t()).reshape(B * S, H)
        eff = self.eff
        h, _ = eff.rms_norm_residual(x, None, w["norm1"], self.eps)
        if d == 128:
            qkv = eff.linear_rope(h, w["wqkv"], cos, sin, hq + hk)   # qkv GEMM with RoPE on q and k in its epilogue
        else:
            qkv = torch.mm(h.view(B * S, H), w["wqkv"].t()).view(B, S, hq + 2 * hk, d)
            eff.rope(qkv[:, :, :hq + hk], cos, sin, None, True)   # q and k heads are neighbours: one launch
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
        if kv_out is not None:
            kv_out[0][:, :, :S].copy_(k.transpose(1, 2))
            kv_out[1][:, :, :S].copy_(v.transpose(1, 2))
        att, _ = eff.sdpa_flash(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), True)
        return torch.mm(att.transpose(1, 2).reshape(B * S, hq * d), w["wo"].t())

    # ---- the same two halves, from already normalised activations (the fused exchange path) ----
    def attn_from_normed(self, h, B, S, out, kv_out=None):
        """h (B*S, hidden): RMS-normalised input of every row. qkv -> RoPE -> attention -> o_proj; this
        rank's partial product (all rows) goes into `out` (B*S, hidden)."""
        hq, hk, d, w = self.hq, self.hk, self.head_dim, self.w
        H = self.hidden
        cos, sin = self.tables(S)
        if self.backend != "gcu":   # plain torch (the host-side test of the schedule)
            qkv = (h.float() @ w["wqkv"].float().t()).view(B, S, hq + 2 * hk, d)
            q = _rope_cpu(qkv[:, :, :hq], cos, sin).transpose(1, 2)
            k = _rope_cpu(qkv[:, :, hq:hq + hk], cos, sin).transpose(1, 2)
            v = qkv[:, :, hq + hk:].transpose(1, 2)
            if kv_out is not None:
                kv_out[0][:, :, :S].copy_(k)
                kv_out[1][:, :, :S].copy_(v)
            g = hq // hk
            att = F.scaled_dot_product_attention(q, k.repeat_interleave(g, 1), v.repeat_interleave(g, 1), is_causal=True)
            out.copy_((att.transpose(1, 2).reshape(B * S, hq * d) @ w["wo"].float().t()).to(out.dtype))
            return
        att = self.attn_core(*self.attn_qkv(h, B, S, kv_out))
        self.attn_out(att, B, S, out)

    # the three launches of the attention part, separately (the exchange schedule treats the attention kernel,
    # which fills an SM's registers on its own, differently from the two projections)
    def attn_qkv(self, h, B, S, kv_out=None):
        hq, hk, d, w, eff, H = self.hq, self.hk, self.head_dim, self.w, self.eff, self.hidden
        cos, sin = self.tables(S)
        if d == 128:
            qkv = eff.linear_rope(h.view(B, S, H), w["wqkv"], cos, sin, hq + hk)
        else:
            qkv = torch.mm(h, w["wqkv"].t()).view(B, S, hq + 2 * hk, d)
            eff.rope(qkv[:, :, :hq + hk], cos, sin, None, True)
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
        if kv_out is not None:
            kv_out[0][:, :, :S].copy_(k.transpose(1, 2))
            kv_out[1][:, :, :S].copy_(v.transpose(1, 2))
        return q, k, v

    def attn_core(self, q, k, v):
        att, _ = self.eff.sdpa_flash(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), True)
        return att

    def attn_out(self, att, B, S, out):
        torch.mm(att.transpose(1, 2).reshape(B * S, self.hq * self.head_dim), self.w["wo"].t(), out=out)

    def mlp_from_normed(self, h2, out):
        """h2 (rows, hidden) normalised: gate/up + SwiGLU -> down; this rank's partial product into `out`."""
        if self.backend != "gcu":
            gu = h2.float() @ self.w["wgu"].float().t()
            out.copy_(((F.silu(gu[..., :self.f]) * gu[..., self.f:]) @ self.w["wd"].float().t()).to(out.dtype))
            return
        act = self.eff.linear_swiglu(h2, self.w["wgu"])
        torch.mm(act, self.w["wd"].t(), out=out)

    def decode_attn_from_normed(self, h, kv, pos, out):
        """One new token per sequence, h (B, hidden) normalised: qkv -> RoPE -> cache update -> attention over
        [0, pos] -> o_proj partial into `out` (B, hidden)."""
        B, H = h.shape
        hq, hk, d, w = self.hq, self.hk, self.head_dim, self.w
        cos, sin = self.tables(kv[0].shape[2])
        if self.backend != "gcu":
            qkv = (h.float() @ w["wqkv"].float().t()).view(B, 1, hq + 2 * hk, d)
            positions = self._positions(B, pos)
            q = _rope_cpu(qkv[:, :, :hq], cos, sin, positions).transpose(1, 2)
            kv[0][:, :, pos:pos + 1].copy_(_rope_cpu(qkv[:, :, hq:hq + hk], cos, sin, positions).transpose(1, 2))
            kv[1][:, :, pos:pos + 1].copy_(qkv[:, :, hq + hk:].transpose(1, 2))
            g = hq // hk
            att = F.scaled_dot_product_attention(q, kv[0][:, :, :pos + 1].float().repeat_interleave(g, 1),
                                                 kv[1][:, :, :pos + 1].float().repeat_interleave(g, 1), is_causal=False)
            out.copy_((att.transpose(1, 2).reshape(B, hq * d) @ w["wo"].float().t()).to(out.dtype))
            return
        eff = self.eff
        qkv = torch.mm(h, w["wqkv"].t()).view(B, 1, hq + 2 * hk, d)
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
        # q rotated in place, rotated k and v written into the cache slot: one launch
        eff.rope_kv_append(qkv, cos, sin, self._positions(B, pos), hq, kv[0], kv[1])
        att, _ = eff.sdpa_flash(q.transpose(1, 2), kv[0][:, :, :pos + 1], kv[1][:, :, :pos + 1], False)
        torch.mm(att.transpose(1, 2).reshape(B, hq * d), w["wo"].t(), out=out)

    def mlp_part(self, o, x):
        """o: the reduced attention output. Returns (down, r): this rank's partial MLP output
        (with the residual already added when tp == 1) and the residual stream."""
        B, S, H = x.shape
        w = self.w
        if self.backend != "gcu":
            r = x.float() + o.view(B, S, H)
            h2 = _rms_cpu(r, w["norm2"], self.eps)
            gu = h2 @ w["wgu"].float().t()
            down = ((F.silu(gu[..., :self.f]) * gu[..., self.f:]) @ w["wd"].float().t()).reshape(B * S, H)
            return (down.view(B, S, H) + r, r) if self.tp == 1 else (down, r)
        eff = self.eff
        h2, r = eff.rms_norm_residual(o.view(B, S, H), x, w["norm2"], self.eps)
        act = eff.linear_swiglu(h2.view(B * S, H), w["wgu"])   # gate/up GEMM with the SwiGLU in its epilogue
        if self.tp == 1:
            return torch.addmm(r.view(B * S, H), act, w["wd"].t()).view(B, S, H), r   # residual in the epilogue
        return torch.mm(act, w["wd"].t()), r

    def forward_prefill(self, x, group=None, kv_out=None):
        B, S, H = x.shape
        o = self.attn_part(x, kv_out)
        self._allreduce(o, group)
        down, r = self.mlp_part(o, x)
        if self.tp == 1:
            return down
        self._allreduce(down, group)
        return torch.add(down.view(B, S, H), r)

    # -------------------------------------------------------------- decode --
    def forward_decode(self, x, kv, pos, group=None):
        """One new token per sequence: x (B,1,hidden); kv = (k_cache, v_cache), each
        (B, kv_heads/tp, T, D); the new K/V rows go to position `pos`, attention
        covers [0, pos]."""
        B, _, H = x.shape
        hq, hk, d, w = self.hq, self.hk, self.head_dim, self.w
        cos, sin = self.tables(kv[0].shape[2])
        assert self.backend == "gcu"
        eff = self.eff
        h, _ = eff.rms_norm_residual(x, None, w["norm1"], self.eps)
        qkv = torch.mm(h.view(B, H), w["wqkv"].t()).view(B, 1, hq + 2 * hk, d)
        q, k, v = qkv[:, :, :hq], qkv[:, :, hq:hq + hk], qkv[:, :, hq + hk:]
        positions = self._positions(B, pos)
        eff.rope_kv_append(qkv, cos, sin, positions, hq, kv[0], kv[1])   # q in place, rotated k and v into the cache slot
        att, _ = eff.sdpa_flash(q.transpose(1, 2), kv[0][:, :, :pos + 1], kv[1][:, :, :pos + 1], False)
        o = torch.mm(att.transpose(1, 2).reshape(B, hq * d), w["wo"].t())
        self._allreduce(o, group)
        h2, r = eff.rms_norm_residual(o.view(B, 1, H), x, w["norm2"], self.eps)
        act = eff.linear_swiglu(h2.view(B, H), w["wgu"])
        if self.tp == 1:
            return torch.addmm(r.view(B, H), act, w["wd"].t()).view(B, 1, H)
        down = torch.mm(act, w["wd"].t())
        self._allreduce(down, group)
        return torch.add(down.view(B, 1, H), r)

    def _positions(self, B, pos):
        key = ("pos", B, pos)
        if key not in self._tables:
            p = torch.full((B, 1), pos, dtype=torch.int64)
            self._tables[key] = p.to(self.device) if self.device is not None else p
        return self._tables[key]


class DecoderStack:
    """`n_layers` layers with independent random-init weights (seed = layer index)."""

    def __init__(self, n_layers, tp, rank, backend, device, dtype, cfg):
        import workloads
        self.layers = [DecoderLayer(workloads.decoder_layer_weights(seed=i, dtype=dtype, tp=tp, rank=rank, **cfg), tp,
                                    backend, device=device, **cfg) for i in range(n_layers)]
        self.cfg, self.tp = cfg, tp
        self._exchanges, self._side_streams = {}, {}
        self.timeline = None   # set to a list to collect (phase, microbatch, start, end) events of eager exchange passes

    # ---- the exchange over peer memory (default for tp > 1 on the device) -----------------------
    def uses_peer_exchange(self):
        """tp > 1 on the device: the row-parallel projections are reduced by this backend's own kernels over
        peer memory (fused with the residual add and the RMSNorm), not by all-reduces of the collective
        library. TP_DECODER_EXCHANGE=nccl keeps the all-reduce path (the comparison)."""
        import os
        return self.tp > 1 and self.layers[0].backend == "gcu" and os.environ.get("TP_DECODER_EXCHANGE", "peer") != "nccl"

    def _exchange(self, key, rows, scatter, group):
        if key not in self._exchanges:
            dtype = self.layers[0].w["wo"].dtype
            if self.layers[0].backend != "gcu":
                self._exchanges[key] = HostExchange(rows, self.cfg["hidden"], dtype, group, scatter=scatter)
            else:
                from torch_gcu.distributed.tp_exchange import TensorParallelExchange
                self._exchanges[key] = TensorParallelExchange(rows, self.cfg["hidden"], dtype, group, scatter=scatter)
        return self._exchanges[key]

    def _prefill_exchange_program(self, x, m, group, caches, result):
        """One microbatch x (B, S, hidden), sequence-parallel between the projections: this rank keeps the
        residual stream of its own 1 / tp of the rows; per projection pair one fused kernel reduces the
        partial products of all ranks for those rows, adds the residual, normalises and scatters the rows
        to every rank, which the next column-parallel projection then reads locally.

        A generator: before every phase it yields the phase's kind -- "compute" (a projection: it wants the
        SMs, and its blocks leave room for exchange blocks beside them), "attention" (the flash kernel: one
        block takes an SM's whole register file) or "exchange" (signal / wait and the fused kernel: they want
        the links) -- and the caller resumes it on the microbatch's stream and uses the kinds to interleave
        the microbatches. The output lands in result[m].

        Why single buffers are safe here (every `sync` is signal + wait = a barrier over the ranks):
        * `partial[k]` is overwritten by this rank's next projection only after the barrier that follows the
          reduce kernel in which the peers read it (a peer signals that barrier after its reduce kernel);
        * `gathered` is overwritten by the peers' next reduce kernel only after the barrier that follows this
          rank's projection that read it (this rank signals that barrier after the projection);
        * the barrier at the top of a pass keeps a fast rank from pushing rows of the next pass into `gathered`
          while a slow rank still copies the previous result out of it."""
        B, S, H = x.shape
        M = B * S
        ex = self._exchange(("prefill", m, M), M, True, group)
        tl = self.timeline   # None, or a list that takes (phase, microbatch, start event, end event)

        def phase(name, fn):
            if tl is None:
                return fn()
            s = torch.gcu.current_stream().record_event(torch.gcu.Event(enable_timing=True))
            r = fn()
            tl.append((name, m, s, torch.gcu.current_stream().record_event(torch.gcu.Event(enable_timing=True))))
            return r

        def exchange(partial, weight, eps, normalise=True):
            phase("wait", ex.sync)         # the partial products are complete on every rank (or: the buffers are free)
            phase("exchange", lambda: ex.reduce_norm(partial, xl, None if partial is None else xl, weight, eps, normalise))
            phase("wait", ex.sync)         # every rank's rows have landed here

        yield "compute"
        xl = x.reshape(M, H)[ex.row0:ex.row0 + ex.rows].clone()   # this rank's rows of the residual stream
        yield "exchange"
        exchange(None, self.layers[0].w["norm1"], self.layers[0].eps)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            kv = None if caches is None else caches[i]
            if layer.backend != "gcu":
                yield "compute"
                layer.attn_from_normed(ex.gathered, B, S, ex.partial[0], kv)
            else:
                yield "compute"
                qkv = phase("attention part", lambda: layer.attn_qkv(ex.gathered, B, S, kv))
                yield "attention"
                att = phase("attention part", lambda: layer.attn_core(*qkv))
                yield "compute"
                phase("attention part", lambda: layer.attn_out(att, B, S, ex.partial[0]))
            yield "exchange"
            exchange(0, layer.w["norm2"], layer.eps)
            yield "compute"
            phase("mlp part", lambda: layer.mlp_from_normed(ex.gathered, ex.partial[1]))
            yield "exchange"
            if i + 1 < n:
                exchange(1, self.layers[i + 1].w["norm1"], self.layers[i + 1].eps)
            else:
                exchange(1, None, 0.0, normalise=False)   # the last residual rows, gathered as they are
        yield "compute"
        result[m] = ex.gathered.clone().view(B, S, H)

    def prefill_exchange(self, x, group, caches=None):
        """Prefill with the peer-memory exchange. The batch is cut into microbatches on streams of their own
        (TP_DECODER_MICROBATCHES, default 2). Their compute phases are chained through events in a fixed
        order (attention part of microbatch 0, of microbatch 1, mlp part of 0, of 1, ...), so each has the SMs
        to itself, and the exchange phase that follows a compute phase runs under the NEXT compute phase of
        the other microbatch: the exchange kernels are small blocks that share the SMs with a resident GEMM
        block. Left to themselves two streams fall into step (both compute, then both exchange) and hide
        nothing. (Measured at four ranks: two free-running streams 14.9 ms per pass, the chain 14.6 ms; also
        keeping the attention kernel, whose blocks fill an SM's register file, apart from the other
        microbatch's exchange: 15.8 ms -- the extra waits cost more than the interference they remove. Compute
        phases on high-priority streams and exchange phases on normal ones, so that a GEMM's blocks are placed
        before the exchange blocks that became ready with it: 15.6 ms, no better either.)"""
        import os
        n_mb = int(os.environ.get("TP_DECODER_MICROBATCHES", "2"))
        if n_mb < 1 or x.shape[0] % n_mb != 0:
            n_mb = 1
        part = x.shape[0] // n_mb
        result = [None] * n_mb

        def kv_of(m):
            return None if caches is None else [tuple(c[m * part:(m + 1) * part] for c in layer_kv) for layer_kv in caches]
        programs = [self._prefill_exchange_program(x[m * part:(m + 1) * part], m, group, kv_of(m), result) for m in range(n_mb)]
        if self.layers[0].backend != "gcu":   # host ranks: the same microbatches and phases, no streams
            for prog in programs:
                for _ in prog:
                    pass
            return result[0] if n_mb == 1 else torch.cat(result, 0)
        main = torch.gcu.current_stream()
        streams = [main]
        for m in range(1, n_mb):
            if m not in self._side_streams:
                self._side_streams[m] = torch.gcu.Stream()
            streams.append(self._side_streams[m])
        fork = main.record_event()
        for s in streams[1:]:
            s.wait_event(fork)
        kinds = [next(prog) for prog in programs]   # the kind of every microbatch's first phase; nothing has run yet
        chain = None                                # completion of the compute / attention phase issued last, on whichever stream
        live = n_mb
        while live:
            for m in range(n_mb):
                if kinds[m] is None:
                    continue
                s = streams[m]
                kind = kinds[m]
                with torch.gcu.stream(s):
                    if kind != "exchange" and chain is not None:
                        s.wait_event(chain)
                    try:
                        kinds[m] = next(programs[m])   # runs the phase that was announced, announces the next
                    except StopIteration:
                        kinds[m] = None
                        live -= 1
                    if kind != "exchange":
                        chain = s.record_event()
        for s in streams[1:]:
            main.wait_event(s.record_event())
        return result[0] if n_mb == 1 else torch.cat(result, 0)

    def decode_exchange(self, x, caches, pos, group):
        """One decode step with the peer-memory exchange: few rows, so every rank reduces all of them for
        itself (one kernel per projection pair that pulls the other ranks' partial rows, adds the residual and
        normalises); the residual stream stays replicated and nothing is gathered.

        Two partial buffers alternate because nothing is gathered here, so no wait orders a peer's read of this
        rank's o_proj partial before this rank's down projection writes: the down projection writes `partial[1]`
        instead. `partial[0]` is rewritten by the next layer's o_proj, which runs after this rank has waited for the
        peers' "down partial ready" signal, and a peer sends that only after its read of `partial[0]`; the same
        argument, one phase later, covers `partial[1]` (also across the end of a step)."""
        B, _, H = x.shape
        ex = self._exchange(("decode", B), B, False, group)
        r = x.view(B, H)
        rbuf = torch.empty_like(r)
        ex.reduce_norm(None, r, None, self.layers[0].w["norm1"], self.layers[0].eps)
        n = len(self.layers)
        for i, (layer, kv) in enumerate(zip(self.layers, caches)):
            layer.decode_attn_from_normed(ex.gathered, kv, pos, ex.partial[0])
            ex.sync()
            ex.reduce_norm(0, r, rbuf, layer.w["norm2"], layer.eps)
            r = rbuf
            layer.mlp_from_normed(ex.gathered, ex.partial[1])
            ex.sync()
            if i + 1 < n:
                ex.reduce_norm(1, r, r, self.layers[i + 1].w["norm1"], self.layers[i + 1].eps)
            else:
                ex.reduce_norm(1, r, r, None, normalise=False)
        return ex.gathered.clone().view(B, 1, H)

    def prefill(self, x, group=None, caches=None, overlap=None):
        if overlap is None and self.uses_peer_exchange():
            return self.prefill_exchange(x, group, caches)
        if overlap is None:
            # measured on B200: tp 8 1.40 M tokens/s against 1.14 M for the plain schedule, tp 4 900 k against
            # 835 k; at tp 2 it only pays when the collective is kept to a few SMs (8 channels, 8 reserved
            # SMs: 583 k against 565 k), because its CTAs otherwise take as much from the GEMMs as they hide
            import os
            overlap = os.environ.get("TP_DECODER_OVERLAP", "1") != "0"
        if self.tp > 1 and overlap and x.shape[0] % 2 == 0:
            if self.layers[0].backend != "gcu":
                return self._two_microbatches(x, group, caches)   # the schedule alone (host-side tests)
            return self._prefill_two_microbatches(x, group, caches)
        for i, layer in enumerate(self.layers):
            x = layer.forward_prefill(x, group, None if caches is None else caches[i])
        return x

    def _prefill_two_microbatches(self, x, group, caches):
        """The batch is cut in two halves that walk the layers one phase apart, so that the
        all-reduce of one half (on the process group's own stream) runs under the other half's
        GEMMs and attention. Same arithmetic per row as the unsplit pass."""
        import os
        import torch.distributed as dist
        # the collective's CTAs need SMs of their own next to the persistent GEMM kernels
        reserve = int(os.environ.get("TP_DECODER_COMM_SMS", "8" if self.tp == 2 else "32"))
        before = torch.gcu.get_reserved_sms()
        torch.gcu.set_reserved_sms(reserve)
        try:
            return self._two_microbatches(x, group, caches)
        finally:
            torch.gcu.set_reserved_sms(before)

    def _two_microbatches(self, x, group, caches):
        import os
        import torch.distributed as dist
        n_mb = int(os.environ.get("TP_DECODER_MICROBATCHES", "2"))
        if x.shape[0] % n_mb != 0:
            n_mb = 2
        part = x.shape[0] // n_mb
        xs = [x[m * part:(m + 1) * part] for m in range(n_mb)]
        B, S, H = xs[0].shape
        pending = [None] * n_mb   # all-reduce of the previous layer's MLP output, per part
        carry = [None] * n_mb     # (down, r) that the pending all-reduce completes
        for i, layer in enumerate(self.layers):
            o, wo = [None] * n_mb, [None] * n_mb
            for m in range(n_mb):
                if pending[m] is not None:
                    pending[m].wait()
                    xs[m] = torch.add(carry[m][0].view(B, S, H), carry[m][1])
                kv = None if caches is None else tuple(c[m * part:(m + 1) * part] for c in caches[i])
                o[m] = layer.attn_part(xs[m], kv)
                wo[m] = dist.all_reduce(o[m], group=group, async_op=True)
            for m in range(n_mb):
                wo[m].wait()
                carry[m] = layer.mlp_part(o[m], xs[m])
                pending[m] = dist.all_reduce(carry[m][0], group=group, async_op=True)
        out = []
        for m in range(n_mb):
            pending[m].wait()
            out.append(torch.add(carry[m][0].view(B, S, H), carry[m][1]))
        return torch.cat(out, 0)

    def decode(self, x, caches, pos, group=None):
        if self.uses_peer_exchange():
            return self.decode_exchange(x, caches, pos, group)
        for layer, kv in zip(self.layers, caches):
            x = layer.forward_decode(x, kv, pos, group)
        return x
