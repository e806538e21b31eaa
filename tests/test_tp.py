"""Partitioned (tensor-parallel) mode: sharding identities on one process, the all-reduce wiring
on two gloo ranks (CPU), and -- on a box with two GPUs -- DF11 shards against BF16 shards."""
import copy
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import dfloat11_b200 as df11
from dfloat11_b200 import codec, tp
from oracle import df11_oracle as oracle
from tests.test_model_api import LLAMA_PATTERNS, tiny_llama

BLOCK = LLAMA_PATTERNS[r"model\.layers\.\d+"]


def test_shard_compress_decode_reassemble_is_identity():
    model = tiny_llama()
    layer = model.model.layers[1]
    plan = tp.default_plan(BLOCK)
    assert plan["self_attn.q_proj"] == "column" and plan["mlp.down_proj"] == "row"
    T = 2
    decoded = []
    for rank in range(T):
        shards = [tp.shard_weight(layer.get_submodule(a).weight.data, plan[a], T, rank) for a in BLOCK]
        t = codec.encode_weights([s.flatten() for s in shards])
        out = oracle.decode_c(t["luts"].numpy(), t["encoded_exponent"].numpy(), t["sign_mantissa"].numpy(),
                              t["output_positions"].numpy(), t["gaps"].numpy())
        flat = torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)
        parts = torch.tensor_split(flat, t["split_positions"].tolist())
        decoded.append([p.view(s.shape) for p, s in zip(parts, shards)])
    for i, a in enumerate(BLOCK):
        whole = tp.unshard_weights([decoded[r][i] for r in range(T)], plan[a])
        assert torch.equal(whole, layer.get_submodule(a).weight.data)


def test_compress_model_tp_writes_one_directory_per_rank(tmp_path):
    model = tiny_llama()
    paths = tp.compress_model_tp(model, LLAMA_PATTERNS, str(tmp_path), tp_size=2)
    assert [os.path.basename(p) for p in paths] == ["rank0-of-2", "rank1-of-2"]
    skeleton = tiny_llama(seed=9)
    loaded = df11.DFloat11Model.from_pretrained(str(tmp_path), device="cpu", bfloat16_model=skeleton,
                                                tp_size=2, tp_rank=1)
    q = loaded.model.layers[0].self_attn.q_proj
    o = loaded.model.layers[0].self_attn.o_proj
    assert (q.out_features, q.in_features) == (128, 256) and (o.out_features, o.in_features) == (256, 128)
    n = sum(m.out_features * m.in_features for m in loaded.model.layers[0].weight_injection_modules)
    assert loaded.model.layers[0].sign_mantissa.numel() == n
    assert loaded.lm_head.sign_mantissa.numel() == 512 * 256            # this rank's half of the vocabulary
    assert loaded.model.embed_tokens.sign_mantissa.numel() == 512 * 256
    assert loaded.model.embed_tokens.num_embeddings == 512 and loaded.lm_head.out_features == 512


def _unit_weights_by_oracle(module):
    out = oracle.decode_c(module.luts.numpy(), module.encoded_exponent.numpy(), module.sign_mantissa.numpy(),
                          module.output_positions.numpy(), module.gaps.numpy())
    return torch.from_numpy(out.view(np.int16)).view(torch.bfloat16)


def test_biases_are_sharded_with_their_layers(tmp_path):
    """Column-parallel biases are cut like the rows they belong to, a row-parallel bias lives on
    rank 0 only, and the default loader path (no ``bfloat16_model``) ends up with exactly those."""
    full = tiny_llama(attention_bias=True)
    with torch.no_grad():
        for name, p in full.named_parameters():
            if name.endswith("bias"):
                p.copy_(torch.randn(p.shape).to(torch.bfloat16))
    want = copy.deepcopy(full)
    tp.compress_model_tp(full, LLAMA_PATTERNS, str(tmp_path), tp_size=2)
    for rank in range(2):
        loaded = df11.DFloat11Model.from_pretrained(str(tmp_path), device="cpu", tp_size=2, tp_rank=rank)
        for i, layer in enumerate(loaded.model.layers):
            ref = want.model.layers[i].self_attn
            att = layer.self_attn
            assert torch.equal(att.q_proj.bias.data, ref.q_proj.bias.data.chunk(2)[rank])
            assert torch.equal(att.k_proj.bias.data, ref.k_proj.bias.data.chunk(2)[rank])
            if rank == 0:
                assert torch.equal(att.o_proj.bias.data, ref.o_proj.bias.data)
            else:
                assert att.o_proj.bias is None
            flat = _unit_weights_by_oracle(layer)
            q = flat[:att.q_proj.out_features * att.q_proj.in_features].view(att.q_proj.out_features, -1)
            assert torch.equal(q, ref.q_proj.weight.data.chunk(2, dim=0)[rank])
        emb = _unit_weights_by_oracle(loaded.model.embed_tokens).view(512, 256)
        assert torch.equal(emb, want.model.embed_tokens.weight.data[rank * 512:(rank + 1) * 512])


def _tp_worker(rank, world, port, use_cuda, path, ids, want, q, peer=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), DF11_PEER_ALLREDUCE="1" if peer else "0")
    dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world)
    try:
        if use_cuda:
            torch.cuda.set_device(rank)
            dev = f"cuda:{rank}"
            bf16 = tiny_llama().to(dev)
            tp.apply_tensor_parallel(bf16, LLAMA_PATTERNS, world, rank)
            df = df11.DFloat11Model.from_pretrained(path, device=dev, bfloat16_model=tiny_llama(seed=5),
                                                    tp_size=world, tp_rank=rank)
            with torch.no_grad():
                a = bf16(input_ids=ids.to(dev)).logits
                b = df(input_ids=ids.to(dev)).logits
            if peer:                                            # the kernel really ran, and no wait ran out
                from dfloat11_b200.comm import PeerAllReduce
                inst = PeerAllReduce.get(None, torch.device(dev))
                assert inst is not None and inst.calls > 0
                inst.check()
            q.put((rank, bool(torch.equal(a, b)), float((a.float().cpu() - want).abs().max())))
        else:
            model = tiny_llama(attention_bias=True, bias_seed=3).float()
            tp.apply_tensor_parallel(model, LLAMA_PATTERNS, world, rank)
            assert model.model.embed_tokens.num_embeddings == 1024 // world
            with torch.no_grad():
                got = model(input_ids=ids).logits
            q.put((rank, got.shape[-1] == 1024, float((got - want).abs().max())))
    finally:
        dist.destroy_process_group()


def _run_ranks(world, use_cuda, path=None, peer=False):
    ids = torch.randint(0, 1024, (2, 17), generator=torch.Generator().manual_seed(4))
    ref = tiny_llama(attention_bias=True, bias_seed=3).float() if not use_cuda else tiny_llama()
    with torch.no_grad():
        want = ref(input_ids=ids).logits.float()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300
    procs = [ctx.Process(target=_tp_worker, args=(r, world, port, use_cuda, path, ids, want, q, peer))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


def test_all_reduce_wiring_on_two_gloo_ranks():
    results = _run_ranks(2, use_cuda=False)
    assert [r[0] for r in results] == [0, 1]
    for _, gathered, err in results:                # fp32 on CPU: only the summation order differs
        assert gathered and err < 1e-3              # full-vocabulary logits on every rank


def _peer_worker(rank, world, port, q):
    """The one-kernel all-reduce against an fp32 sum of the same inputs, eagerly, back to back
    (call parity, counters) and replayed from a CUDA graph."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from dfloat11_b200.comm import PeerAllReduce
        inst = PeerAllReduce.get(None, dev)
        if inst is None:
            q.put((rank, "unavailable"))
            return
        ok = True
        for n in (8, 16384, 16384, 40000, 16 * 16384, 16384):
            parts = [torch.randn(n, generator=torch.Generator().manual_seed(100 * n + r)).to(torch.bfloat16)
                     for r in range(world)]
            want = torch.zeros(n)
            for p in parts:                                  # rank order, fp32, one rounding: what the kernel does
                want = want + p.float()
            x = parts[rank].to(dev)
            assert inst.all_reduce_(x)
            ok &= bool(torch.equal(x.cpu(), want.to(torch.bfloat16)))
        assert not inst.all_reduce_(torch.zeros(7, dtype=torch.bfloat16, device=dev))      # not a multiple of 8
        assert not inst.all_reduce_(torch.zeros(8, dtype=torch.float32, device=dev))
        # three calls in one graph, replayed: the call number lives on the device
        x = torch.ones(4096, dtype=torch.bfloat16, device=dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            inst.all_reduce_(x)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        dist.barrier(device_ids=[rank])
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(3):
                inst.all_reduce_(x)
        x.fill_(1.0)
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
        ok &= bool((x == float(world) ** 6).all()) if world <= 2 else True
        inst.check()
        # the call number wraps: the tag of the pushed form skips 0, the buffer halves keep alternating
        torch.cuda.synchronize()
        dist.barrier(device_ids=[rank])
        inst.counters[0] = -3                                  # 0xFFFFFFFD, on every rank, nothing in flight
        inst.counters[2:] = -3                                 # (the pushed form counts per CTA)
        torch.cuda.synchronize()
        dist.barrier(device_ids=[rank])
        for k in range(8):
            x = torch.full((40000 if k % 2 else 16384,), float(rank + 1 + k), dtype=torch.bfloat16, device=dev)  # both forms
            assert inst.all_reduce_(x)
            ok &= bool((x == float(sum(r + 1 + k for r in range(world)))).all())
        ok &= inst.counters[:3].cpu().tolist() == [1, 0, 1]
        inst.check()
        q.put((rank, "ok" if ok else "wrong"))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_all_reduce_kernels_with_all_ranks_on_one_gpu(world):
    """Both forms of the all-reduce kernel with 2, 4 and 8 ranks played by one cooperative launch
    on one GPU: results against an fp32 sum in rank order, the call numbers, the alternating
    buffer halves, and the wrap of the call number."""
    from dfloat11_b200 import _lib
    lib, dev, slot = _lib.lib, torch.device("cuda", 0), 1 << 20
    flag_bytes = int(lib.df11_allreduce_flag_bytes())
    data = torch.zeros(world * 2 * slot, dtype=torch.uint8, device=dev)
    flags = torch.zeros(world * flag_bytes, dtype=torch.uint8, device=dev)
    words = int(lib.df11_allreduce_counter_bytes()) // 4
    counters = torch.zeros(world, words, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def one_call(n, seed):
        parts = torch.randn(world, n, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
        want = torch.zeros(n)
        for r in range(world):                                # rank order, fp32, one rounding
            want = want + parts[r].float()
        x, out = parts.to(dev), torch.empty(world, n, dtype=torch.bfloat16, device=dev)
        _lib.check(lib.df11_selftest_allreduce_one_gpu(world, data.data_ptr(), flags.data_ptr(), counters.data_ptr(),
                                                       x.data_ptr(), out.data_ptr(), n, slot, 0, status.data_ptr(),
                                                       0, stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        for r in range(world):
            assert torch.equal(out[r].cpu(), want.to(torch.bfloat16)), (n, r)

    sizes = (8, 16384, 16384, 40000, 32768, 16 * 16384, 40000, 16384, 1000 * 8)   # pushed form up to 32768 elements
    pushed = flagged = 0
    for k, n in enumerate(sizes):
        one_call(n, 17 * k + world)
        takes_pushed = n <= 32768 and world != 3               # 3 ranks: the general kernel, flag form only
        pushed, flagged = pushed + takes_pushed, flagged + (not takes_pushed)
        # [0] calls of the flag form, [1] its CTAs done, [2 + c] pushed calls CTA c took part in
        assert counters[:, :3].cpu().tolist() == [[flagged, 0, pushed]] * world
    assert counters[:, 2 + 31].cpu().tolist() == [int(world != 3)] * world   # only the 32768-element call reached the last CTA
    counters[:, 0] = -3                                       # 0xFFFFFFFD: the tags pass 0xFFFFFFFF, skip 0
    counters[:, 2:] = -3
    torch.cuda.synchronize()
    for k in range(8):
        one_call(40000 if k % 2 else 16384, 900 + k)
    assert counters[:, :3].cpu().tolist() == ([[1, 0, 1]] if world != 3 else [[5, 0, -3]]) * world
    with pytest.raises(_lib.DF11Error):
        _lib.check(lib.df11_selftest_allreduce_one_gpu(5, data.data_ptr(), flags.data_ptr(), counters.data_ptr(),
                                                       data.data_ptr(), data.data_ptr(), 8, slot, 0, status.data_ptr(),
                                                       0, stream))


@pytest.mark.gpu
def test_all_reduce_gives_up_when_a_peer_never_comes():
    """Rank 0 of two on one GPU, the other rank's buffers standing by untouched: nothing ever sets
    its tags or flags, so the wait (50 ms here) runs out, the status word says so and the kernel
    returns; while the status is set the next call does not wait again.  Both forms."""
    import ctypes
    import time
    from dfloat11_b200 import _lib
    lib, dev, slot = _lib.lib, torch.device("cuda", 0), 1 << 20
    flag_bytes = int(lib.df11_allreduce_flag_bytes())
    buffers = [torch.zeros(2 * slot + flag_bytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    data = (ctypes.c_uint64 * 8)(*([b.data_ptr() for b in buffers] + [0] * 6))
    flags = (ctypes.c_uint64 * 8)(*([b.data_ptr() + 2 * slot for b in buffers] + [0] * 6))
    counters = torch.zeros(int(lib.df11_allreduce_counter_bytes()) // 4, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call(x, wait_ms):
        torch.cuda.synchronize()
        t0 = time.time()
        _lib.check(lib.df11_allreduce_bf16(data, flags, counters.data_ptr(), 0, 2, x.data_ptr(), x.data_ptr(),
                                           x.numel(), slot, wait_ms, status.data_ptr(), 0, stream))
        torch.cuda.synchronize()
        return time.time() - t0

    for n in (16384, 40000):                                   # pushed form, flag form
        x = torch.ones(n, dtype=torch.bfloat16, device=dev)
        waited = call(x, 50)
        assert int(status.item()) & _lib.STATUS_TIMEOUT
        assert 0.04 < waited < 5.0
        assert call(x, 5000) < 1.0                             # gave up before: no second wait
        status.zero_()
    assert counters[:3].cpu().tolist() == [2, 0, 2]            # the call numbers went on all the same


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2])
def test_peer_all_reduce_kernel(world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs more GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 300 + world
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=300) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    if any(r[1] == "unavailable" for r in results):
        pytest.skip("symmetric memory cannot be set up on this box")
    assert [r[1] for r in results] == ["ok"] * world


@pytest.mark.gpu
@pytest.mark.parametrize("peer", [False, True])
def test_df11_shards_match_bf16_shards_on_two_gpus(tmp_path, peer):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    tp.compress_model_tp(tiny_llama(), LLAMA_PATTERNS, str(tmp_path), tp_size=2)
    results = _run_ranks(2, use_cuda=True, path=str(tmp_path), peer=peer)
    for _, identical, err in results:
        assert identical                            # same TP degree: bit-identical logits
        assert err < 0.25                           # and close to the unsharded BF16 model
