"""Seeded synthetic inputs for the benchmark configurations.

Every tensor is drawn on the CPU from `torch.Generator().manual_seed(seed)` in
the fixed order written here and only then copied to the device, so the GPU
kernels and the CPU ATen baseline see identical bits. bf16 tensors are made by
rounding the fp32 draw. Nothing here comes from a dataset: "Llama-style" fixes
shapes only.
"""
import torch


def _gen(seed):
    g = torch.Generator()
    g.manual_seed(seed)
    return g


def op_sweep(rows=4096, cols=4096, seed=0):
    """fp32 (rows, cols) ~ N(0,1): add, mul, silu, casts, sum, softmax, layer_norm."""
    g = _gen(seed)
    a = torch.randn(rows, cols, generator=g)
    b = torch.randn(rows, cols, generator=g)
    w = torch.randn(cols, generator=g) * 0.02 + 1.0
    bias = torch.randn(cols, generator=g) * 0.02
    return dict(a=a, b=b, weight=w, bias=bias, eps=1e-5)


def index_ops(vocab=128256, hidden=4096, batch=8, seq=2048, n_select=65536, gather_rows=8192,
              gather_cols=1024, scatter_src=262144, scatter_dst=65536, scatter_cols=256, seed=0):
    """Embedding / index_select on one bf16 table; gather; scatter_add / index_put rows."""
    g = _gen(seed)
    table = (torch.randn(vocab, hidden, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (batch, seq), generator=g, dtype=torch.int64)
    select_idx = torch.randint(0, vocab, (n_select,), generator=g, dtype=torch.int64)
    gather_src = torch.randn(gather_rows, gather_cols, generator=g)
    gather_idx = torch.randint(0, gather_cols, (gather_rows, gather_cols), generator=g, dtype=torch.int64)
    scatter_vals = torch.randn(scatter_src, scatter_cols, generator=g)
    scatter_rows = torch.randint(0, scatter_dst, (scatter_src,), generator=g, dtype=torch.int64)
    return dict(table=table, ids=ids, select_idx=select_idx, gather_src=gather_src, gather_idx=gather_idx,
                scatter_vals=scatter_vals, scatter_rows=scatter_rows, scatter_dst=scatter_dst,
                scatter_cols=scatter_cols)


def rope_tables(seq, head_dim, theta=10000.0):
    """fp32 cos/sin tables (seq, head_dim/2): pos * theta^(-2i/D), the HF recipe."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(seq, dtype=torch.float32), inv_freq)
    return freqs.cos().contiguous(), freqs.sin().contiguous()


def fused_ops(tokens=16384, hidden=4096, batch=8, seq=2048, heads=32, kv_heads=8, head_dim=128,
              ffn=14336, seed=0):
    g = _gen(seed)
    bf = torch.bfloat16
    x = torch.randn(tokens, hidden, generator=g).to(bf)
    res = torch.randn(tokens, hidden, generator=g).to(bf)
    w = (torch.randn(hidden, generator=g) * 0.02 + 1.0).to(bf)
    q = torch.randn(batch, seq, heads, head_dim, generator=g).to(bf)
    k = torch.randn(batch, seq, kv_heads, head_dim, generator=g).to(bf)
    gate = torch.randn(tokens, ffn, generator=g).to(bf)
    up = torch.randn(tokens, ffn, generator=g).to(bf)
    cos, sin = rope_tables(seq, head_dim)
    return dict(x=x, res=res, weight=w, eps=1e-6, q=q, k=k, gate=gate, up=up, cos=cos, sin=sin)


def decoder_layer_weights(hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336, seed=0,
                          dtype=torch.bfloat16, tp=1, rank=0):
    """Random-init N(0, 0.02) weights of one Llama-style layer, optionally the
    tensor-parallel shard of `rank` (column-parallel q/k/v/gate/up, row-parallel
    o/down). Every rank draws the full matrices from the same seed and slices, so
    shards are consistent across ranks."""
    g = _gen(seed)
    def mat(o, i):
        return torch.randn(o, i, generator=g) * 0.02
    wq, wk, wv = mat(heads * head_dim, hidden), mat(kv_heads * head_dim, hidden), mat(kv_heads * head_dim, hidden)
    wo = mat(hidden, heads * head_dim)
    wg, wu = mat(ffn, hidden), mat(ffn, hidden)
    wd = mat(hidden, ffn)
    n1 = torch.randn(hidden, generator=g) * 0.02 + 1.0
    n2 = torch.randn(hidden, generator=g) * 0.02 + 1.0
    if tp > 1:
        hq, hk, f = heads // tp * head_dim, kv_heads // tp * head_dim, ffn // tp
        wq, wk, wv = wq[rank * hq:(rank + 1) * hq], wk[rank * hk:(rank + 1) * hk], wv[rank * hk:(rank + 1) * hk]
        wo = wo[:, rank * hq:(rank + 1) * hq]
        wg, wu = wg[rank * f:(rank + 1) * f], wu[rank * f:(rank + 1) * f]
        wd = wd[:, rank * f:(rank + 1) * f]
    out = dict(wqkv=torch.cat([wq, wk, wv], 0), wo=wo.contiguous(), wgu=torch.cat([wg, wu], 0),
               wd=wd.contiguous(), norm1=n1, norm2=n2)
    return {k: v.to(dtype).contiguous() for k, v in out.items()}
