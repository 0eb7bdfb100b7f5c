"""One forward pass worth of the hot-path ops, in model order, on one GPU's shard of the tokens.

Per pass and per token the reference engine runs (engine.py:254-272 with the
block bodies in model/{mamba,attention,mlp}_block.cuh): one embedding gather,
42 pre-norm RMSNorms each preceded by the previous block's residual add, 21
gated RMSNorms inside the Mamba-2 blocks and 17 relu^2 inside the MLP blocks.
With the add fused into the norm that follows it this is 1 + 42 + 21 + 17 = 81
launches.  The GEMMs, scans and attention between them are not part of this
library; their outputs are stood in for by resident synthetic tensors (the
"mixer outputs"), which is also how the ops see them in the engine: as bf16
tensors already in device memory.

Every op is independent per token row, so N GPUs each run the same chain on
their own rows with no exchange: `shard_range` gives rank k its rows.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import ops

HIDDEN = 3136
D_INNER = 6144            # width of the gated RMSNorm in the benchmark configuration
N_GROUPS = 8
INTER = 12544
VOCAB = 131072
N_LAYERS = 42


def layer_schedule() -> str:
    """42 layers: 'M' Mamba-2 (21), '-' MLP (17), '*' attention (4), interleaved like a hybrid stack."""
    pat = "M-M-M-M-M*" * 4 + "M-"
    assert len(pat) == N_LAYERS and pat.count("M") == 21 and pat.count("-") == 17 and pat.count("*") == 4
    return pat


def shard_range(total_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [lo, hi) that rank `rank` of `world` owns: contiguous, balanced to within one row."""
    if world < 1 or not (0 <= rank < world) or total_rows < 0:
        raise ValueError("bad shard request")
    return (rank * total_rows) // world, ((rank + 1) * total_rows) // world


def bytes_per_token(ids_bytes: int = 4) -> int:
    """Algorithmic HBM bytes one token costs per pass (each activation byte crosses HBM once)."""
    gather = 2 * HIDDEN * 2 + ids_bytes
    return gather + 42 * (4 * HIDDEN * 2) + 21 * (3 * D_INNER * 2) + 17 * (2 * INTER * 2)


BATCH_BLOCK_ROWS = 2048   # granularity of the seeded generation of a global batch (see batch_shard)


def batch_shard(global_tokens: int, lo: int, hi: int, device, seed: int = 0, vocab: int = VOCAB,
                ids_dtype=torch.int32, mixer_sets: int = 2) -> dict:
    """Rows [lo, hi) of ONE seeded global batch of `global_tokens` tokens, as the `init` of a ChainPass.

    The batch is defined block by block: rows [k*BATCH_BLOCK_ROWS, (k+1)*BATCH_BLOCK_ROWS) of every
    per-token tensor come from a generator seeded with (seed, tensor, k), so the values of a row do not
    depend on which rank generates it or on how many ranks there are; a rank generates only the blocks
    its rows touch.  The table and the norm weights (replicated on every GPU) have seeds of their own.
    Value distributions are the benchmark configuration's: table 0.02*N(0,1), ids uniform over the
    vocabulary, mixer outputs / y / z N(0,1), u 2*N(0,1), weights 1 + 0.1*N(0,1); generated in fp32 and
    cast to bf16."""
    if not (0 <= lo <= hi <= global_tokens):
        raise ValueError("bad row range")
    dev, bf = torch.device(device), torch.bfloat16

    def gen(tag: int, block: int = 0) -> torch.Generator:
        g = torch.Generator(device=dev)
        g.manual_seed((int(seed) * 1000003 + tag) * 1000003 + block)
        return g

    def rows(tag: int, cols: int, scale: float = 1.0) -> torch.Tensor:
        out = torch.empty(hi - lo, cols, device=dev, dtype=bf)
        for k in range(lo // BATCH_BLOCK_ROWS, -(-hi // BATCH_BLOCK_ROWS) if hi > lo else 0):
            b0 = k * BATCH_BLOCK_ROWS
            n = min(BATCH_BLOCK_ROWS, global_tokens - b0)
            blk = (scale * torch.randn(n, cols, generator=gen(tag, k), device=dev, dtype=torch.float32)).to(bf)
            s0, s1 = max(lo, b0), min(hi, b0 + n)
            out[s0 - lo:s1 - lo] = blk[s0 - b0:s1 - b0]
        return out

    ids = torch.empty(hi - lo, device=dev, dtype=torch.int64)
    for k in range(lo // BATCH_BLOCK_ROWS, -(-hi // BATCH_BLOCK_ROWS) if hi > lo else 0):
        b0 = k * BATCH_BLOCK_ROWS
        n = min(BATCH_BLOCK_ROWS, global_tokens - b0)
        blk = torch.randint(0, vocab, (n,), generator=gen(1, k), device=dev, dtype=torch.int64)
        s0, s1 = max(lo, b0), min(hi, b0 + n)
        ids[s0 - lo:s1 - lo] = blk[s0 - b0:s1 - b0]
    table = torch.empty(vocab, HIDDEN, device=dev, dtype=bf)
    g_t, step = gen(0), 8192
    for r0 in range(0, vocab, step):                 # chunked: keeps the fp32 temporary small
        table[r0:r0 + step] = (0.02 * torch.randn(min(step, vocab - r0), HIDDEN, generator=g_t, device=dev,
                                                  dtype=torch.float32)).to(bf)
    g_w = gen(2)
    norm_w = 1.0 + 0.1 * torch.randn(N_LAYERS, HIDDEN, generator=g_w, device=dev, dtype=torch.float32)
    gated_w = 1.0 + 0.1 * torch.randn(21, D_INNER, generator=g_w, device=dev, dtype=torch.float32)
    return dict(table=table, ids=ids.to(ids_dtype), mixer_out=[rows(10 + j, HIDDEN) for j in range(mixer_sets)],
                y=rows(3, D_INNER), z=rows(4, D_INNER), u=rows(5, INTER, 2.0), norm_w=norm_w, gated_w=gated_w)


@dataclass
class ChainBuffers:
    table: torch.Tensor
    ids: torch.Tensor
    hidden: list            # two [T, HIDDEN] ping-pong buffers (engine.py:70)
    normed: torch.Tensor
    mixer_out: list         # stand-ins for the blocks' GEMM outputs, rotated
    y: torch.Tensor
    z: torch.Tensor
    gated_out: torch.Tensor
    u: torch.Tensor
    act: torch.Tensor
    norm_w: torch.Tensor    # [42, HIDDEN] fp32
    gated_w: torch.Tensor   # [21, D_INNER] fp32
    err_flag: torch.Tensor


class ChainPass:
    """Holds the resident tensors of one shard and enqueues the 81-launch pass."""

    def __init__(self, tokens: int, device, ids_dtype=torch.int32, seed: int = 0, mixer_sets: int = 2,
                 vocab: int = VOCAB, init: dict | None = None):
        self.tokens = int(tokens)
        self.device = torch.device(device)
        self.schedule = layer_schedule()
        T, dev, bf = self.tokens, self.device, torch.bfloat16
        if init is None:
            g = torch.Generator(device=dev)
            g.manual_seed(seed)
            rn = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.float32)  # noqa: E731
            table = torch.empty(vocab, HIDDEN, device=dev, dtype=bf)
            step = 8192
            for lo in range(0, vocab, step):      # chunked: keeps the fp32 temporary small
                table[lo:lo + step] = (0.02 * rn(min(step, vocab - lo), HIDDEN)).to(bf)
            ids = torch.randint(0, vocab, (T,), generator=g, device=dev, dtype=torch.int64).to(ids_dtype)

            def big(cols, scale=1.0):
                out = torch.empty(T, cols, device=dev, dtype=bf)
                rows = max(1, (1 << 26) // cols)
                for lo in range(0, T, rows):
                    out[lo:lo + rows] = (scale * rn(min(rows, T - lo), cols)).to(bf)
                return out
            init = dict(table=table, ids=ids, mixer_out=[big(HIDDEN) for _ in range(mixer_sets)],
                        y=big(D_INNER), z=big(D_INNER), u=big(INTER, 2.0),
                        norm_w=1.0 + 0.1 * rn(N_LAYERS, HIDDEN), gated_w=1.0 + 0.1 * rn(21, D_INNER))
        mk = lambda cols: torch.empty(T, cols, device=dev, dtype=bf)  # noqa: E731
        self.buf = ChainBuffers(
            table=init["table"].to(dev), ids=init["ids"].to(dev),
            hidden=[mk(HIDDEN), mk(HIDDEN)], normed=mk(HIDDEN),
            mixer_out=[t.to(dev) for t in init["mixer_out"]],
            y=init["y"].to(dev), z=init["z"].to(dev), gated_out=mk(D_INNER),
            u=init["u"].to(dev), act=mk(INTER),
            norm_w=init["norm_w"].to(dev).contiguous(), gated_w=init["gated_w"].to(dev).contiguous(),
            err_flag=torch.zeros(1, device=dev, dtype=torch.int32))
        self.launches_per_pass = 1 + 42 + 21 + 17
        self._host_ids = None
        self._host_out = None
        self.graph = None
        self.graph_launches = 0

    def run(self) -> torch.Tensor:
        """Enqueues one pass on torch's current stream; returns the final normed hidden states [T, HIDDEN]."""
        self._enqueue_rows(0, self.tokens)
        return self.buf.normed

    def _enqueue_rows(self, lo: int, hi: int) -> None:
        """The 81 launches on rows [lo, hi) of every resident tensor (tokens are independent: a row range of the
        pass is the pass of that row range)."""
        b = self.buf
        cur, other = b.hidden[0][lo:hi], b.hidden[1][lo:hi]
        mixer = [m[lo:hi] for m in b.mixer_out]
        y, z, gated_out, u, act, normed = b.y[lo:hi], b.z[lo:hi], b.gated_out[lo:hi], b.u[lo:hi], b.act[lo:hi], b.normed[lo:hi]
        ops.embedding(b.table, b.ids[lo:hi], out=cur, err_flag=b.err_flag)
        n_m = 0
        for i, kind in enumerate(self.schedule):
            if kind == "M":
                ops.rmsnorm_gated(y, z, b.gated_w[n_m], D_INNER // N_GROUPS, out=gated_out)
                n_m += 1
            elif kind == "-":
                ops.relu2(u, out=act)
            ops.add_rmsnorm(cur, mixer[i % len(mixer)], b.norm_w[i], out_res=other, out=normed)
            cur, other = other, cur
        self.final_hidden = b.hidden[len(self.schedule) % 2]      # the buffers swap once per layer

    def capture(self) -> None:
        """Records the 81-launch pass into a CUDA graph.  For decode-sized shards (T = 1 ... 64) the pass is
        bound by launch overhead, not bandwidth: one graph launch replaces 81 host-side launches."""
        self.run()                                   # warm-up outside the capture (one-time kernel attributes)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            self.run()
        self.graph = graph
        self.graph_launches = ops.launch_count() - before   # kernel nodes one replay enqueues

    def replay(self) -> torch.Tensor:
        """Replays the captured pass on the current stream; same buffers, same result as run()."""
        self.graph.replay()
        return self.buf.normed

    def capture_pipelined(self, full_output: torch.Tensor, chunks: int) -> None:
        """Records the pass as `chunks` row ranges, each followed by the copy of its normed rows to `full_output`
        (pinned host memory) on a second stream, so that a range travels to the host while the next one is computed.
        One graph; `full_output` must be the same tensor on every replay."""
        T = self.tokens
        bounds = [shard_range(T, c, chunks) for c in range(chunks)]
        side = torch.cuda.Stream(device=self.device)
        self.run()                                   # one-time kernel attributes, outside the capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            main = torch.cuda.current_stream()
            for lo, hi in bounds:
                if hi <= lo:
                    continue
                self._enqueue_rows(lo, hi)
                done = torch.cuda.Event()
                done.record(main)
                side.wait_event(done)
                with torch.cuda.stream(side):
                    full_output[lo:hi].copy_(self.buf.normed[lo:hi], non_blocking=True)
            joined = torch.cuda.Event()
            joined.record(side)
            main.wait_event(joined)
        self._pipe = (graph, full_output.data_ptr(), chunks)

    def run_from_host(self, ids_host: torch.Tensor, full_output: torch.Tensor | None = None, chunks: int | None = None) -> torch.Tensor:
        """The end-to-end call: token ids arrive in (pinned) host memory, the last token's normed hidden
        state comes back to host memory — what the engine's prefill hands to lm_head (engine.py:241-251).
        The pass is the captured graph when capture() has been called, host-launched otherwise.  With
        `full_output` (a pinned [T, HIDDEN] bf16 host tensor) every normed row is copied back instead: in `chunks`
        row ranges whose copies overlap the next range's kernels (default: 4 ranges from 32,768 tokens up, else 1)."""
        b = self.buf
        if self._host_out is None:
            self._host_out = torch.empty(HIDDEN, dtype=torch.bfloat16).pin_memory()
        b.ids.copy_(ids_host, non_blocking=True)
        if full_output is not None:
            if chunks is None:
                chunks = 4 if self.tokens >= 32768 else 1
            if chunks > 1 and full_output.is_pinned():
                pipe = getattr(self, "_pipe", None)
                if pipe is None or pipe[1] != full_output.data_ptr() or pipe[2] != chunks:
                    self.capture_pipelined(full_output, chunks)
                    b.ids.copy_(ids_host, non_blocking=True)
                self._pipe[0].replay()
                torch.cuda.current_stream().synchronize()
                return full_output
        normed = self.replay() if getattr(self, "graph", None) is not None else self.run()
        if full_output is not None:
            full_output.copy_(normed, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return full_output
        self._host_out.copy_(normed[self.tokens - 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._host_out
