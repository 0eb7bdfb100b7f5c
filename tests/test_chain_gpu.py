"""The 81-launch per-pass op mix on the GPU against the same chain evaluated with the CPU oracle."""
import pytest
import torch

from oracle import torch_golden as og

pytestmark = pytest.mark.gpu


def oracle_chain(chain_mod, init, schedule):
    hidden = og.embedding(init["ids"], init["table"])
    n_m, gated, act, normed = 0, None, None, None
    for i, kind in enumerate(schedule):
        if kind == "M":
            gated = og.gated_rmsnorm_bf16(init["y"], init["z"], init["gated_w"][n_m], chain_mod.D_INNER // chain_mod.N_GROUPS)
            n_m += 1
        elif kind == "-":
            act = og.relu2_bf16(init["u"])
        hidden, normed = og.add_rmsnorm_bf16(hidden, init["mixer_out"][i % len(init["mixer_out"])], init["norm_w"][i])
    return hidden, normed, gated, act


@pytest.mark.parametrize("T", [1, 257])
def test_chain_pass_matches_oracle(built_lib, T):
    from nemotron_infer_b200 import chain, ops
    built_lib.nmt_set_device(torch.cuda.current_device())
    g = torch.Generator().manual_seed(11)
    bf = torch.bfloat16
    vocab = 1024
    init = dict(
        table=(0.02 * torch.randn(vocab, chain.HIDDEN, generator=g)).to(bf),
        ids=torch.randint(0, vocab, (T,), generator=g, dtype=torch.int64).to(torch.int32),
        mixer_out=[torch.randn(T, chain.HIDDEN, generator=g).to(bf) for _ in range(2)],
        y=torch.randn(T, chain.D_INNER, generator=g).to(bf), z=torch.randn(T, chain.D_INNER, generator=g).to(bf),
        u=(2 * torch.randn(T, chain.INTER, generator=g)).to(bf),
        norm_w=1 + 0.1 * torch.randn(chain.N_LAYERS, chain.HIDDEN, generator=g),
        gated_w=1 + 0.1 * torch.randn(21, chain.D_INNER, generator=g))
    cp = chain.ChainPass(T, "cuda", vocab=vocab, init=init)
    before = ops.launch_count()
    normed = cp.run()
    torch.cuda.synchronize()
    assert ops.launch_count() - before == 81 == cp.launches_per_pass
    want_hidden, want_normed, want_gated, want_act = oracle_chain(chain, init, cp.schedule)
    assert torch.equal(cp.final_hidden.cpu().view(torch.int16), want_hidden.view(torch.int16)), "residual stream must be bit-exact"
    assert og.ulp_report(normed, want_normed)["max_ulp"] <= 1
    assert og.ulp_report(cp.buf.gated_out, want_gated)["max_ulp"] <= 1
    assert torch.equal(cp.buf.act.cpu().view(torch.int16), want_act.view(torch.int16))
    assert int(cp.buf.err_flag.item()) == 0
    # the end-to-end call (host ids in, last token's normed state out) returns the same row
    host_ids = init["ids"].clone().pin_memory()
    out = cp.run_from_host(host_ids)
    assert og.ulp_report(out, want_normed[T - 1])["max_ulp"] <= 1


def test_graph_replay_equals_eager_pass(built_lib):
    """The captured CUDA graph of the pass (decode-sized shard) reproduces the host-launched pass bit for bit,
    with programmatic dependent launch on or off."""
    from nemotron_infer_b200 import chain, ops
    for T in (1, 64):
        cp = chain.ChainPass(T, "cuda", vocab=4096, seed=T)
        ref = cp.run().clone()
        ref_hidden = cp.final_hidden.clone()
        try:
            for pdl in (2, 1):                      # 2 = plain launches, 1 = programmatic dependent launch
                ops.tune("launch.pdl", pdl)
                assert torch.equal(cp.run().view(torch.int16), ref.view(torch.int16))
                cp.capture()
                cp.buf.normed.zero_()
                got = cp.replay()
                torch.cuda.synchronize()
                assert torch.equal(got.view(torch.int16), ref.view(torch.int16))
                assert torch.equal(cp.final_hidden.view(torch.int16), ref_hidden.view(torch.int16))
        finally:
            ops.tune("launch.pdl", 0)
    assert built_lib.nmt_device_wait_timeouts() == 0


def test_sharded_chain_equals_unsharded(built_lib):
    """Token sharding: running rows [lo, hi) alone gives exactly the rows of the full run (no cross-row term)."""
    from nemotron_infer_b200 import chain
    T, vocab = 96, 512
    g = torch.Generator().manual_seed(5)
    bf = torch.bfloat16
    full = dict(
        table=(0.02 * torch.randn(vocab, chain.HIDDEN, generator=g)).to(bf),
        ids=torch.randint(0, vocab, (T,), generator=g, dtype=torch.int64).to(torch.int32),
        mixer_out=[torch.randn(T, chain.HIDDEN, generator=g).to(bf) for _ in range(2)],
        y=torch.randn(T, chain.D_INNER, generator=g).to(bf), z=torch.randn(T, chain.D_INNER, generator=g).to(bf),
        u=(2 * torch.randn(T, chain.INTER, generator=g)).to(bf),
        norm_w=1 + 0.1 * torch.randn(chain.N_LAYERS, chain.HIDDEN, generator=g),
        gated_w=1 + 0.1 * torch.randn(21, chain.D_INNER, generator=g))
    whole = chain.ChainPass(T, "cuda", vocab=vocab, init=full)
    ref = whole.run().clone()
    world = 4
    for rank in range(world):
        lo, hi = chain.shard_range(T, rank, world)
        part = {k: (v[lo:hi] if k in ("ids", "y", "z", "u") else v) for k, v in full.items()}
        part["mixer_out"] = [m[lo:hi] for m in full["mixer_out"]]
        got = chain.ChainPass(hi - lo, "cuda", vocab=vocab, init=part).run()
        assert torch.equal(got.view(torch.int16), ref[lo:hi].view(torch.int16))


def test_bench_parity_sample_and_batch_shards(built_lib):
    """bench.py's own output check (sampled rows of the pass against the oracle) passes on a correct pass and
    notices a corrupted one; the ranks' shards of one seeded batch give the rows of the whole batch."""
    import bench
    from nemotron_infer_b200 import chain
    G, vocab = 300, 2048
    whole = chain.ChainPass(G, "cuda", init=chain.batch_shard(G, 0, G, "cuda", seed=8, vocab=vocab))
    ref = whole.run().clone()
    rep = bench.parity_sample(whole, 64, seed=1)
    assert rep["max_ulp"] <= 1 and rep["not_bit_exact"] == [] and rep["err_flag"] == 0 and rep["rows"] >= 32
    assert sorted(rep["bit_exact"]) == ["act", "final_hidden"]
    for rank in range(3):
        lo, hi = chain.shard_range(G, rank, 3)
        part = chain.ChainPass(hi - lo, "cuda", init=chain.batch_shard(G, lo, hi, "cuda", seed=8, vocab=vocab))
        assert torch.equal(part.run().view(torch.int16), ref[lo:hi].view(torch.int16))
    # the captured pass serves the host-buffer call, and a full-output request returns every row
    whole.capture()
    ids_host = whole.buf.ids.cpu().pin_memory()
    rows_host = torch.empty(G, chain.HIDDEN, dtype=torch.bfloat16).pin_memory()
    last = whole.run_from_host(ids_host).clone()
    assert torch.equal(last.view(torch.int16), ref[G - 1].cpu().view(torch.int16))
    assert torch.equal(whole.run_from_host(ids_host, full_output=rows_host).view(torch.int16), ref.cpu().view(torch.int16))
    assert whole.graph_launches == 81
    # ... also as three row ranges whose copies to the host overlap the next range's kernels (one graph, two streams)
    rows_host.zero_()
    launches = built_lib.nmt_launch_count()
    got = whole.run_from_host(ids_host, full_output=rows_host, chunks=3)
    assert built_lib.nmt_launch_count() - launches == 81 + 3 * 81          # one warm-up pass, then three ranges captured
    assert torch.equal(got.view(torch.int16), ref.cpu().view(torch.int16))
    rows_host.zero_()
    assert torch.equal(whole.run_from_host(ids_host, full_output=rows_host, chunks=3).view(torch.int16), ref.cpu().view(torch.int16))
    assert torch.equal(whole.final_hidden.view(torch.int16), whole.buf.hidden[0].view(torch.int16))
    # a wrong byte in the residual stream or the activation is reported
    whole.final_hidden[0, 0] += 1.0
    whole.buf.normed[G - 1, 5] = 1000.0
    bad = bench.parity_sample(whole, 64, seed=1)
    assert "final_hidden" in bad["not_bit_exact"] and bad["max_ulp"] > 1
