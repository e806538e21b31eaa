"""Loader, hook, buffer manager, offload and model API (mirrors of dfloat11/dfloat11.py).

CPU tests cover the file format round trip (``compress_model`` -> safetensors + config ->
``load_and_replace_tensors``) with every unit decoded by the CPU oracle; GPU tests check that a
DF11 model produces logits bit-identical to the uncompressed BF16 model, with and without
``cpu_offload``, through ``DFloat11Model.from_pretrained``.
"""
import copy
import json
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

import dfloat11_b200 as df11
from dfloat11_b200 import dfloat11 as host
from dfloat11_b200.placement import infer_device_map, module_bytes
from oracle import df11_oracle as oracle

LLAMA_PATTERNS = {
    r"model\.embed_tokens": [],
    r"model\.layers\.\d+": ["self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
                             "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj"],
    r"lm_head": [],
}


def tiny_llama(seed=0, attention_bias=False, bias_seed=None):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=256, intermediate_size=704, num_hidden_layers=3, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=1024, max_position_embeddings=256,
                      tie_word_embeddings=False, attention_bias=attention_bias)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_((torch.randn(p.shape) * (1.0 if "embed" in name else 0.02)).to(torch.bfloat16))
        if bias_seed is not None:                       # q/k/v/o biases (the Qwen2 layout), seeded
            g = torch.Generator().manual_seed(bias_seed)
            for name, p in model.named_parameters():
                if name.endswith("bias"):
                    p.copy_((torch.randn(p.shape, generator=g) * 0.1).to(torch.bfloat16))
    return model


@pytest.fixture
def seek16():
    """Rows of 512 elements are whole chunks only with a seek point every 16 elements."""
    before = df11.seek_interval()
    df11.seek_interval(16)
    yield
    df11.seek_interval(before)


@pytest.fixture(scope="module")
def saved(tmp_path_factory):
    model = tiny_llama()
    reference = copy.deepcopy(model)
    path = str(tmp_path_factory.mktemp("df11_llama"))
    df11.compress_model(model, LLAMA_PATTERNS, path, save_single_file=False, check_correctness=False)
    return path, reference


def test_compress_model_writes_the_reference_layout(saved):
    path, reference = saved
    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    assert "model_layers_0.safetensors" in files and "lm_head.safetensors" in files
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)["dfloat11_config"]
    assert cfg["bytes_per_thread"] == 8 and list(cfg["threads_per_block"]) == [512]
    assert set(cfg["pattern_dict"]) == set(LLAMA_PATTERNS)
    from safetensors.torch import load_file
    t = load_file(os.path.join(path, "model_layers_1.safetensors"))
    direct = {k[len("model.layers.1."):] for k in t if k.count(".") == 3}
    assert direct == {"luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps", "split_positions"}
    assert "model.layers.1.input_layernorm.weight" in t          # the block's own small tensors travel with it
    assert not any(k.endswith("proj.weight") for k in t)
    assert t["model.layers.1.output_positions"].dtype == torch.uint8
    assert t["model.layers.1.split_positions"].dtype == torch.int64
    # the stored unit decodes (CPU oracle) to the original seven matrices, in order
    out = oracle.decode_c(*(t[f"model.layers.1.{k}"].numpy() for k in
                            ("luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps")))
    layer = reference.model.layers[1]
    want = torch.cat([layer.get_submodule(a).weight.detach().flatten() for a in LLAMA_PATTERNS[r"model\.layers\.\d+"]])
    assert np.array_equal(out, want.view(torch.int16).numpy().view(np.uint16))


def test_loader_arms_units_on_cpu(saved):
    path, reference = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cpu", bfloat16_model=tiny_llama(seed=7))
    layer = model.model.layers[0]
    for name in ("luts", "encoded_exponent", "sign_mantissa", "output_positions", "gaps"):
        assert name in dict(layer.named_buffers(recurse=False))
    assert isinstance(layer.split_positions, list) and len(layer.split_positions) == 6
    assert len(layer.weight_injection_modules) == 7
    assert not hasattr(layer.self_attn.q_proj, "weight")
    assert not hasattr(model.lm_head, "weight") and not hasattr(model.model.embed_tokens, "weight")
    assert layer.max_block_elems > 0 and layer.shared_mem_size == 2052 + 2 * layer.max_block_elems
    # uncompressed tensors (norms) were copied from the file, not left at the skeleton's values
    assert torch.equal(model.model.norm.weight, reference.model.norm.weight)
    # without a GPU the hook refuses to run instead of falling back to something else
    with pytest.raises(RuntimeError):
        model(torch.zeros(1, 4, dtype=torch.long))


def test_loader_offload_keeps_big_tensors_on_host(saved):
    path, _ = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cpu", bfloat16_model=tiny_llama(seed=7),
                                               cpu_offload=True, cpu_offload_blocks=2, pin_memory=False)
    offloaded = [m for m in model.modules() if hasattr(m, "offloaded_tensors")]
    assert len(offloaded) == 2                                   # cpu_offload_blocks limits the count
    for m in offloaded:
        assert set(m.offloaded_tensors) == {"encoded_exponent", "sign_mantissa"}
        assert "encoded_exponent" not in dict(m.named_buffers(recurse=False))
        assert m.df11_next_offloaded in offloaded


def test_loader_rejects_corrupt_units(saved, tmp_path):
    path, _ = saved
    from safetensors.torch import load_file, save_file
    t = load_file(os.path.join(path, "lm_head.safetensors"))
    t["lm_head.luts"] = t["lm_head.luts"].clone()
    t["lm_head.luts"][-1] = 0                                     # zero code lengths
    bad = str(tmp_path / "bad.safetensors")
    save_file(t, bad)
    skeleton = nn.Module()
    skeleton.lm_head = nn.Linear(256, 1024, bias=False).to(torch.bfloat16)
    with pytest.raises(RuntimeError):
        df11.DFloat11Model.from_single_file(bad, pattern_dict={r"lm_head": []}, bfloat16_model=skeleton, device="cpu")


def test_missing_config_and_paths(tmp_path, saved):
    with pytest.raises(FileNotFoundError):
        df11.DFloat11Model.from_pretrained(str(tmp_path / "nope.safetensors"), from_single_file=True,
                                           bfloat16_model=nn.Linear(2, 2))
    with pytest.raises(IsADirectoryError):
        df11.DFloat11Model.from_pretrained(str(tmp_path), from_single_file=True, bfloat16_model=nn.Linear(2, 2))
    (tmp_path / "config.json").write_text("{}")
    with pytest.raises(AttributeError):
        df11.DFloat11Model.from_pretrained(str(tmp_path), bfloat16_model=nn.Linear(2, 2), device="cpu")


def test_get_hook_rejects_other_layouts():
    with pytest.raises(ValueError):
        host.get_hook((256,), 8)


def test_no_split_classes_and_device_map(saved):
    path, _ = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cpu", bfloat16_model=tiny_llama(seed=7))
    classes = df11.get_no_split_classes(model, LLAMA_PATTERNS)
    assert "LlamaDecoderLayer" in classes and "Linear" in classes and "Embedding" in classes
    mapping = infer_device_map(model, classes, devices=[0, 1])
    assert {str(d) for d in mapping.values()} == {"cuda:0", "cuda:1"}
    # a compressed block is never divided and blocks fill devices in order
    layer_devs = [mapping[f"model.layers.{i}"] for i in range(3)]
    assert layer_devs == sorted(layer_devs, key=lambda d: d.index)
    assert not any(k.startswith("model.layers.0.") for k in mapping)
    assert module_bytes(model) == sum(module_bytes(model.get_submodule(k)) for k in mapping)


def test_tensor_manager_reuses_and_grows():
    host.TensorManager.release()
    a = host.TensorManager.allocate_bfloat16("cpu", 100)
    b = host.TensorManager.allocate_bfloat16("cpu", 60)
    assert b.data_ptr() == a.data_ptr() and b.numel() == 60
    c = host.TensorManager.allocate_bfloat16("cpu", 500)
    assert c.numel() == 500 and host.TensorManager._tensors[(torch.device("cpu"), 0)].numel() == 500
    d = host.TensorManager.allocate_bfloat16("cpu", 40, slot=1)            # slots are separate tensors
    assert d.data_ptr() != c.data_ptr() and host.TensorManager.allocate_bfloat16("cpu", 10).data_ptr() == c.data_ptr()
    host.TensorManager.release("cpu")
    assert not host.TensorManager._tensors
    # the largest unit that is decoded whole sizes slots 0 / 1 at their first allocation
    host.TensorManager.min_elements = 300
    e = host.TensorManager.allocate_bfloat16("cpu", 100)
    assert e.numel() == 100 and host.TensorManager._tensors[(torch.device("cpu"), 0)].numel() == 300
    assert host.TensorManager.allocate_bfloat16("cpu", 7, slot=2).numel() == 7
    assert host.TensorManager._tensors[(torch.device("cpu"), 2)].numel() == 7
    host.TensorManager.release()
    assert host.TensorManager.min_elements == 0


def test_growing_the_scratch_takes_back_the_views_of_the_old_one():
    host.TensorManager.release()
    layer = nn.Linear(4, 3, bias=False)
    del layer._parameters["weight"]
    layer.split_positions = []
    small = host.TensorManager.allocate_bfloat16("cpu", 12)
    host._inject_weights(layer, small)
    assert layer.weight.shape == (3, 4) and layer.weight.data_ptr() == small.data_ptr()
    host.TensorManager.allocate_bfloat16("cpu", 1000)           # grows: the old tensor must not stay referenced
    assert layer.weight is None and layer.__dict__["df11_injected"] is None
    host.TensorManager.release()


def test_environment_switches_are_read_once_per_forward_of_a_marked_model(monkeypatch):
    net = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    host._mark_root(net)
    host._mark_root(net)                                         # idempotent
    seen = []
    net[0].register_forward_pre_hook(lambda mod, inp: seen.append((host._use_fused_gemv(), host._Flags.in_forward)))

    def flip(mod, inp):                                          # a change in mid-forward is not seen before the next one
        monkeypatch.setenv("DF11_FUSED_GEMV", "0")
        seen.append((host._use_fused_gemv(), host._Flags.in_forward))
    net[1].register_forward_pre_hook(flip)
    monkeypatch.setenv("DF11_FUSED_GEMV", "1")
    net(torch.zeros(1, 2))
    net(torch.zeros(1, 2))
    assert seen == [(True, True), (True, True), (False, True), (False, True)]
    assert host._Flags.in_forward is False
    monkeypatch.setenv("DF11_FUSED_GEMV", "1")                   # outside a forward: read on every call
    assert host._use_fused_gemv()
    monkeypatch.setenv("DF11_FUSED_GEMV", "0")
    assert not host._use_fused_gemv()
    with pytest.raises(RuntimeError):                            # an exception in the forward still ends it
        net(torch.zeros(1, 3))
    assert host._Flags.in_forward is False


def test_placement_moves_structured_outputs_and_keeps_their_type():
    from collections import namedtuple
    from transformers import DynamicCache
    from transformers.modeling_outputs import CausalLMOutputWithPast
    from dfloat11_b200.placement import _first_tensor_device, _move
    cpu = torch.device("cpu")
    out = CausalLMOutputWithPast(logits=torch.zeros(1, 2, 3), past_key_values=DynamicCache())
    moved = _move(out, cpu)
    assert type(moved) is CausalLMOutputWithPast and moved.logits is out.logits
    assert moved.past_key_values is out.past_key_values           # objects that are not tensors pass through
    pair = namedtuple("pair", "a b")(torch.zeros(1), [torch.ones(2), {"k": torch.ones(1)}])
    moved = _move(pair, cpu)
    assert type(moved) is type(pair) and isinstance(moved.b, list) and isinstance(moved.b[1], dict)
    assert _first_tensor_device((), {"input_ids": torch.zeros(1)}) == cpu
    assert _first_tensor_device((None, [3, (torch.zeros(1),)]), {}) == cpu
    assert _first_tensor_device((1, "x"), {}) is None


def test_fused_product_groups_follow_the_layer_families(seek16):
    """q/k/v and gate/up of a block are served by one stacked product each; o and down stand alone;
    a unit whose rows are not multiples of 512 elements, a lookup table or an offloaded unit take no
    fused product at all."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=1, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=1024, max_position_embeddings=64, tie_word_embeddings=False)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    df11.compress_in_place(model, LLAMA_PATTERNS)
    block = model.model.layers[0]
    layers = host._fused_layers(block)
    assert [first for _, first in layers] == [0] + list(block.split_positions)
    groups = host._fused_groups(block, layers)
    names = {id(m): n.rsplit(".", 1)[-1] for n, m in block.named_modules()}
    assert [[names[id(l)] for l, _ in g] for g in groups] == [["q_proj", "k_proj", "v_proj"], ["o_proj"],
                                                              ["gate_proj", "up_proj"], ["down_proj"]]
    assert host._fused_layers(model.model.embed_tokens) is None
    assert [first for _, first in host._fused_layers(model.lm_head)] == [0]
    small = tiny_llama()                                         # hidden 256: rows of 256 elements
    df11.compress_in_place(small, LLAMA_PATTERNS)
    assert host._fused_layers(small.model.layers[0]) is None
    block.offloaded_tensors = {}
    assert host._fused_layers(block) is None


def test_from_pretrained_builds_its_own_skeleton(saved):
    """The call the reference's README shows: only a path.  The skeleton comes from the saved
    ``config.json`` (AutoConfig -> from_config without weight initialisation, dfloat11.py:409-419),
    ``dfloat11_config`` is read from that same file, ordinary tensors (norms) come from what
    ``save_pretrained`` wrote beside the units (dfloat11.py:600-604,619-622)."""
    path, reference = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cpu")
    assert type(model).__name__ == "LlamaForCausalLM" and not model.training
    assert model.config.dfloat11_config["bytes_per_thread"] == 8
    ref_params = dict(reference.named_parameters())
    seen = 0
    for name, p in model.named_parameters():                     # what is left are the uncompressed tensors
        assert p.dtype == torch.bfloat16 and torch.equal(p.data, ref_params[name].data), name
        seen += 1
    assert seen == 2 * 3 + 1                                      # two norms per layer and the final norm
    for name, unit in [("model.layers.2", model.model.layers[2]), ("lm_head", model.lm_head)]:
        out = oracle.decode_c(unit.luts.numpy(), unit.encoded_exponent.numpy(), unit.sign_mantissa.numpy(),
                              unit.output_positions.numpy(), unit.gaps.numpy())
        ref_unit = reference.get_submodule(name)
        want = torch.cat([p.data.flatten() for _, p in ref_unit.named_parameters() if p.dim() == 2])
        assert np.array_equal(out.view(np.int16), want.view(torch.int16).numpy()), name
        assert not any(n.endswith("weight") and p.dim() == 2 for n, p in unit.named_parameters())


def test_graphed_decoder_refuses_a_model_that_is_not_on_a_gpu():
    with pytest.raises(RuntimeError):
        df11.GraphedGreedyDecoder(nn.Linear(2, 2))


# ------------------------------------------------------------------ GPU
@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["resident", "ahead", "ahead_3_ctas", "ahead_window", "offload", "offload_some_ahead", "two_pass",
                                  "auto_map"])
def test_logits_identical_to_bf16_model(saved, mode, monkeypatch):
    path, reference = saved
    kwargs = dict(device="cuda:0")
    host._DecodeAhead._by_device.clear()
    if "ahead" in mode:
        monkeypatch.setenv("DF11_DECODE_AHEAD", "1")             # next unit decoded on a second stream
    if mode == "ahead_3_ctas":
        monkeypatch.setenv("DF11_AHEAD_CTAS", "3")
    if mode == "ahead_window":                                   # part of the next unit beside attention, the rest in its own hook
        monkeypatch.setenv("DF11_DECODE_AHEAD", "2")
    if mode == "offload":
        kwargs["cpu_offload"] = True
    elif mode.startswith("offload_some"):
        kwargs.update(cpu_offload=True, cpu_offload_blocks=2)
    elif mode == "two_pass":
        monkeypatch.setenv("DF11_PREPARED", "0")
    elif mode == "auto_map":
        kwargs = dict(device=None, device_map="auto")
    model = df11.DFloat11Model.from_pretrained(path, bfloat16_model=tiny_llama(seed=7), **kwargs)
    ref = copy.deepcopy(reference).to("cuda:0")
    ids = torch.randint(0, 1024, (2, 33), generator=torch.Generator().manual_seed(3)).to("cuda:0")
    with torch.no_grad():
        for _ in range(3):                      # several forwards: scratch and staging slots are reused
            got = model(input_ids=ids).logits
            want = ref(input_ids=ids).logits
            assert torch.equal(got, want)
        out_a = model.generate(ids[:1, :8], max_new_tokens=12, do_sample=False)
        out_b = ref.generate(ids[:1, :8], max_new_tokens=12, do_sample=False)
    assert torch.equal(out_a, out_b)
    if mode.startswith("offload"):
        stager = host._OffloadStager.get(torch.device("cuda:0"))
        assert stager.stats["prefetch_hits"] > 0 and stager.stats["h2d_bytes"] > 0
    ahead = host._DecodeAhead._by_device.get(torch.device("cuda:0"))
    if "ahead" in mode:
        # from the second forward on, resident units are decompressed while their predecessor computes
        assert ahead is not None and ahead.stats["hits"] > 0 and ahead.pending is None
    else:
        assert ahead is None or ahead.stats["launched"] == 0


@pytest.mark.gpu
def test_switching_decode_ahead_off_again_keeps_the_weights_right(saved, monkeypatch):
    """The short path of the hook keeps pointers and weight views from a unit's last call; a pass
    in another mode (here: decode-ahead, whose units alternate between two scratch tensors)
    re-injects the views, and the short path must not trust its old state afterwards."""
    path, reference = saved
    host._DecodeAhead._by_device.clear()
    model = df11.DFloat11Model.from_pretrained(path, bfloat16_model=tiny_llama(seed=7), device="cuda:0")
    ref = copy.deepcopy(reference).to("cuda:0")
    ids = torch.randint(0, 1024, (2, 19), generator=torch.Generator().manual_seed(5)).to("cuda:0")
    with torch.no_grad():
        want = ref(input_ids=ids).logits
        for setting in (None, None, "1", "1", None, None, "2", "2", None, None):
            if setting is None:
                monkeypatch.delenv("DF11_DECODE_AHEAD", raising=False)
            else:
                monkeypatch.setenv("DF11_DECODE_AHEAD", setting)
            assert torch.equal(model(input_ids=ids).logits, want), setting


@pytest.mark.gpu
@pytest.mark.parametrize("offload", [False, True])
def test_from_pretrained_without_a_skeleton_gives_bf16_logits(saved, offload):
    """Default branch of ``from_pretrained`` (no ``bfloat16_model``) end to end on the GPU."""
    from transformers import AutoConfig, AutoModelForCausalLM
    path, reference = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cuda:0", cpu_offload=offload)
    # the uncompressed model built the same way (from the saved config, in BF16 from the start: its
    # rotary tables stay fp32, where `tiny_llama()` rounds them to BF16 with the rest of the model)
    ref = AutoModelForCausalLM.from_config(AutoConfig.from_pretrained(path), dtype=torch.bfloat16)
    ref.load_state_dict(reference.state_dict())
    ref = ref.eval().to("cuda:0")
    ids = torch.randint(0, 1024, (2, 21), generator=torch.Generator().manual_seed(11)).to("cuda:0")
    with torch.no_grad():
        for _ in range(2):
            assert torch.equal(model(input_ids=ids).logits, ref(input_ids=ids).logits)
        assert torch.equal(model.generate(ids[:1, :6], max_new_tokens=10, do_sample=False),
                           ref.generate(ids[:1, :6], max_new_tokens=10, do_sample=False))


@pytest.mark.gpu
def test_status_word_stats_and_nvtx_switch(saved, monkeypatch):
    """Every launch of the hooks reports into one status word per device: a forward over tensors
    that went bad raises from ``check_status`` (or by itself with DF11_CHECK_STATUS=1) instead of
    silently computing with unspecified weights; ``stats()`` counts what the hooks did."""
    path, reference = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cuda:0", bfloat16_model=tiny_llama(seed=7))
    ids = torch.randint(0, 1024, (1, 12), generator=torch.Generator().manual_seed(3)).to("cuda:0")
    before = df11.stats()
    monkeypatch.setenv("DF11_NVTX", "1")                      # the slower, fully checked path with ranges around it
    with torch.no_grad():
        model(input_ids=ids)
        monkeypatch.setenv("DF11_NVTX", "0")
        model(input_ids=ids)
    after = df11.stats()
    assert after["decodes"] >= before["decodes"] + 2 * 4 and after["decoded_elements"] > before["decoded_elements"]
    assert any(k.startswith("cuda:0/slot0") for k in after["scratch_bytes"])
    df11.check_status()                                       # nothing wrong so far
    layer = model.model.layers[1]
    good = layer.luts.clone()
    layer.luts[-1, :] = 0                                     # code lengths of 0: the reference kernel would spin on these
    layer.__dict__.pop("df11_aux", None)                      # rebuild the tables from the broken luts
    layer.__dict__["df11_fast"] = None
    with torch.no_grad():
        model(input_ids=ids)
    with pytest.raises(df11._lib.DF11Error):
        df11.check_status()
    df11.check_status()                                       # the word was reset by the failed check
    monkeypatch.setenv("DF11_CHECK_STATUS", "1")
    with torch.no_grad(), pytest.raises(df11._lib.DF11Error):
        model(input_ids=ids)
    layer.luts.copy_(good)
    layer.__dict__.pop("df11_aux", None)
    with torch.no_grad():
        model(input_ids=ids)                                  # repaired: the per-forward check passes again


@pytest.mark.gpu
def test_compress_model_self_check_and_single_file(tmp_path):
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(384, 640, bias=True)
            self.b = nn.Linear(640, 384, bias=False)

        def forward(self, x):
            return self.b(torch.relu(self.a(x)))

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList([Block() for _ in range(2)])
            self.head = nn.Linear(384, 10)

        def forward(self, x):
            for blk in self.blocks:
                x = x + blk(x)
            return self.head(x)

    torch.manual_seed(1)
    net = Net().to(torch.bfloat16).eval()
    reference = copy.deepcopy(net).to("cuda:0")
    patterns = {r"blocks\.\d+": ["a", "b"], r"head": []}
    df11.compress_model(net, patterns, str(tmp_path), save_single_file=True, check_correctness=True)
    torch.manual_seed(2)
    loaded = df11.DFloat11Model.from_single_file(os.path.join(str(tmp_path), "model.safetensors"), patterns,
                                                 Net().to(torch.bfloat16).eval(), device="cuda:0")
    x = torch.randn(5, 384, dtype=torch.bfloat16, device="cuda:0")
    with torch.no_grad():
        assert torch.equal(loaded(x), reference(x))


@pytest.mark.gpu
def test_embedding_unit_decodes_only_looked_up_rows(tmp_path, monkeypatch, seek16):
    torch.manual_seed(5)
    emb = nn.Embedding(2000, 512).to(torch.bfloat16)
    reference = copy.deepcopy(emb).to("cuda:0")
    holder = nn.Module()
    holder.emb = emb
    ref_holder = nn.Module()
    df11.compress_model(holder, {r"emb": []}, str(tmp_path), save_single_file=True, check_correctness=True)
    skeleton = nn.Module()
    skeleton.emb = nn.Embedding(2000, 512).to(torch.bfloat16)
    loaded = df11.DFloat11Model.from_single_file(os.path.join(str(tmp_path), "model.safetensors"), {r"emb": []},
                                                 skeleton, device="cuda:0")
    ids = torch.randint(0, 2000, (3, 9), device="cuda:0")
    with torch.no_grad():
        got = loaded.emb(ids)
        assert loaded.emb.weight.shape == (27, 512)               # only the looked-up rows were decoded
        assert torch.equal(got, reference(ids))
        big = torch.randint(0, 2000, (4, 600), device="cuda:0")   # more lookups than rows: whole table
        got = loaded.emb(big)
        assert loaded.emb.weight.shape == (2000, 512)
        assert torch.equal(got, reference(big))
        monkeypatch.setenv("DF11_SPARSE_EMBEDDING", "0")
        assert torch.equal(loaded.emb(ids), reference(ids))
        assert loaded.emb.weight.shape == (2000, 512)
    del ref_holder


def _wide_llama(seed=0):
    """Hidden size 1024 (rows that every seek interval can cut), a vocabulary of 16384."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=1024, intermediate_size=2048, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=8, vocab_size=16384, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(seed)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_((torch.randn(p.shape) * (1.0 if "embed" in name else 0.02)).to(torch.bfloat16))
    return model


@pytest.mark.gpu
@pytest.mark.parametrize("offload", [False, True])
def test_large_head_is_multiplied_slab_by_slab(monkeypatch, offload):
    """A single-Linear unit above SLAB_MIN_ELEMENTS called with up to four activation vectors is
    decompressed and multiplied in slabs of rows inside the scratch sized for the transformer
    blocks; logits stay bit-identical to BF16 and the scratch never grows to the size of the head.
    Under cpu_offload the embedding's rows are read straight from pinned memory (never staged)."""
    monkeypatch.setattr(host, "SLAB_MIN_ELEMENTS", 1 << 22)              # the 16384 x 1024 head counts as large
    host.TensorManager.release()
    host._OffloadStager._by_device.clear()
    model = _wide_llama().to("cuda:0")
    ref = copy.deepcopy(model)
    df11.compress_in_place(model, LLAMA_PATTERNS, cpu_offload=offload)
    head_elements = 16384 * 1024
    block_elements = 4 * 1024 * 1024 + 3 * 1024 * 2048
    assert host.TensorManager.min_elements == block_elements
    assert model.lm_head.__dict__.get("df11_slabbed") and 0 < host._slab_rows(model.lm_head) < 16384
    before = df11.stats()["slab_products"]
    dev = torch.device("cuda:0")
    with torch.no_grad():
        for tokens in (1, 3, 4):
            ids = torch.randint(0, 16384, (1, tokens), generator=torch.Generator().manual_seed(tokens)).to(dev)
            assert torch.equal(model(input_ids=ids).logits, ref(input_ids=ids).logits)
        assert df11.stats()["slab_products"] == before + 3
        assert host.TensorManager._tensors[(dev, 0)].numel() == block_elements < head_elements
        out_a = model.generate(ids[:, :1], max_new_tokens=6, do_sample=False)
        assert torch.equal(out_a, ref.generate(ids[:, :1], max_new_tokens=6, do_sample=False))
        ids = torch.randint(0, 16384, (2, 9), generator=torch.Generator().manual_seed(9)).to(dev)
        assert torch.equal(model(input_ids=ids).logits, ref(input_ids=ids).logits)      # 18 vectors: whole decode
        assert host.TensorManager._tensors[(dev, 0)].numel() >= head_elements
        ids = ids[:1, :2]
        assert torch.equal(model(input_ids=ids).logits, ref(input_ids=ids).logits)      # and slabs again afterwards
        monkeypatch.setenv("DF11_SLAB_HEAD", "0")
        assert torch.equal(model(input_ids=ids).logits, ref(input_ids=ids).logits)
    df11.check_status()
    if offload:
        staged = host._OffloadStager.get(dev).stats["h2d_bytes"]
        emb = model.model.embed_tokens.offloaded_tensors
        assert staged > 0 and "df11_next_offloaded" not in model.model.embed_tokens.__dict__
        assert all(s["owner"] is not model.model.embed_tokens for s in host._OffloadStager.get(dev).slots)
        assert emb["sign_mantissa"].is_pinned() and model.model.embed_tokens.weight.shape[0] <= 18
    block = model.model.layers[0]
    if offload:          # bound by its host -> device copy: self-contained kernel, no auxiliary buffer on the device
        assert block.__dict__.get("df11_aux") is None and block.gaps.is_cuda
        assert model.lm_head.__dict__.get("df11_aux") is not None        # the slab-wise head keeps its seek points
    else:                # side tensors parked on the host once the auxiliary buffer exists
        assert block.__dict__.get("df11_aux") is not None and not block.gaps.is_cuda
    host.TensorManager.release()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(151936, 4096), (128256, 4096), (12288, 4096), (4096, 14336)])
def test_row_slabs_of_a_product_have_the_bits_of_the_whole_product(rows, cols):
    """What the slab-wise head relies on: for a few activation vectors the library computes each
    output row the same way whether it is given the whole [rows, cols] matrix or a block of its
    rows -- checked at the baseline configurations' head and MLP shapes, slabs of 47104 rows (a
    Qwen3-8B block's worth of scratch) and of 8192."""
    import torch.nn.functional as F
    g = torch.Generator(device="cuda:0").manual_seed(rows)
    w = (torch.randn(rows, cols, device="cuda:0", generator=g) * 0.02).to(torch.bfloat16)
    for m in (1, 2, 3, 4):
        x = torch.randn(1, m, cols, device="cuda:0", generator=g).to(torch.bfloat16)
        whole = F.linear(x, w)
        for slab in (47104, 8192):
            got = torch.empty_like(whole)
            for r0 in range(0, rows, slab):
                r1 = min(rows, r0 + slab)
                if m == 1:
                    torch.mm(x.view(1, cols), w[r0:r1].t(), out=got.view(1, rows)[:, r0:r1])
                else:
                    got[..., r0:r1] = F.linear(x, w[r0:r1])
            assert torch.equal(got, whole), (m, slab)


@pytest.mark.gpu
def test_fused_products_for_single_token_steps(monkeypatch, seek16):
    """DF11_FUSED_GEMV=1: a forward over a few tokens multiplies straight from the compressed
    weights (same exact products, fp32 sums in another order than the library GEMV: logits
    agree to BF16 rounding, not bit for bit); a longer forward decompresses as usual and stays
    bit-identical."""
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=8,
                      num_key_value_heads=2, vocab_size=1024, max_position_embeddings=256, tie_word_embeddings=False)
    torch.manual_seed(11)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16).eval()
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.copy_((torch.randn(p.shape) * (1.0 if "embed" in name else 0.03)).to(torch.bfloat16))
    reference = copy.deepcopy(model).to("cuda:0")
    model = model.to("cuda:0")
    df11.compress_in_place(model, LLAMA_PATTERNS)
    monkeypatch.setenv("DF11_FUSED_GEMV", "1")
    calls = []
    real = host.ops.gemv_prepared
    monkeypatch.setattr(host.ops, "gemv_prepared", lambda *a, **k: (calls.append(a[5:8]), real(*a, **k))[1])
    ids = torch.randint(0, 1024, (1, 21), generator=torch.Generator().manual_seed(5)).to("cuda:0")
    with torch.no_grad():
        want = reference(input_ids=ids).logits
        got = model(input_ids=ids).logits                         # 21 tokens: ordinary decode
        assert torch.equal(got, want) and not calls
        cache_a = model(input_ids=ids, use_cache=True).past_key_values
        cache_b = reference(input_ids=ids, use_cache=True).past_key_values
        tok = ids[:, -1:]
        got1 = model(input_ids=tok, past_key_values=cache_a, use_cache=True).logits
        want1 = reference(input_ids=tok, past_key_values=cache_b, use_cache=True).logits
    # per block: q/k/v stacked, o, gate/up stacked, down; and the head
    assert len(calls) == 2 * 4 + 1
    assert (0, 512 + 128 + 128, 512) in calls and (0, 1024, 512) in calls and calls.count((393216, 512, 512)) == 2
    scale = float(want1.float().abs().max())
    assert float((got1.float() - want1.float()).abs().max()) <= 0.03 * scale
    assert torch.equal(got1.argmax(-1), want1.argmax(-1))
    monkeypatch.setenv("DF11_FUSED_GEMV", "0")
    with torch.no_grad():                                         # switched off again: the usual path, bit-identical
        again = model(input_ids=ids).logits
    assert torch.equal(again, want)


def _eager_static_greedy(model, ids, n_new, max_cache_len=64):
    """The loop the graphed decoder captures, run eagerly: static KV cache, arg-max per step."""
    from transformers import StaticCache
    cache = StaticCache(config=model.config, max_cache_len=max_cache_len)
    out = [ids]
    with torch.no_grad():
        logits = model(input_ids=ids, past_key_values=cache, cache_position=torch.arange(ids.shape[1], device=ids.device),
                       use_cache=True).logits
        tok = logits[:, -1:].argmax(-1)
        pos = torch.tensor([ids.shape[1]], device=ids.device)
        for _ in range(n_new - 1):
            out.append(tok)
            logits = model(input_ids=tok, past_key_values=cache, cache_position=pos, use_cache=True).logits
            tok = logits[:, -1:].argmax(-1)
            pos = pos + 1
        out.append(tok)
    return torch.cat(out, dim=1)


@pytest.mark.gpu
def test_graphed_greedy_decoder(saved):
    """One CUDA graph per token gives the ids of the same loop run eagerly, for the DF11 model and
    for the BF16 one (which agree with each other), on repeated calls and with an end-of-sequence id."""
    path, reference = saved
    model = df11.DFloat11Model.from_pretrained(path, device="cuda:0", bfloat16_model=tiny_llama(seed=7))
    ref = copy.deepcopy(reference).to("cuda:0")
    ids = torch.randint(0, 1024, (1, 9), generator=torch.Generator().manual_seed(8)).to("cuda:0")
    other = torch.randint(0, 1024, (1, 5), generator=torch.Generator().manual_seed(9)).to("cuda:0")
    want = _eager_static_greedy(ref, ids, 20)
    want_other = _eager_static_greedy(ref, other, 7)
    assert torch.equal(_eager_static_greedy(model, ids, 20), want)
    for m in (model, ref):
        decoder = df11.GraphedGreedyDecoder(m, max_cache_len=64)
        assert torch.equal(decoder.generate(ids, 20), want)
        assert torch.equal(decoder.generate(ids, 20), want)                  # the captured graph is reused
        assert torch.equal(decoder.generate(ids, 1), want[:, :10])
        assert torch.equal(decoder.generate(other, 7), want_other)
        eos = int(want[0, 9 + 6])
        got = decoder.generate(ids, 20, eos_token_id=eos, eos_check_every=4)
        first = int((want[0, 9:] == eos).nonzero()[0])
        assert torch.equal(got, want[:, :9 + first + 1])
    with pytest.raises(ValueError):
        decoder.generate(ids, 100)
    # a batch of prompts: the DF11 model and the BF16 model produce the same ids (a new capture per batch size)
    batch = torch.randint(0, 1024, (3, 9), generator=torch.Generator().manual_seed(10)).to("cuda:0")
    got = [df11.GraphedGreedyDecoder(m, max_cache_len=64).generate(batch, 12) for m in (model, ref)]
    assert got[0].shape == (3, 21) and torch.equal(got[0], got[1]) and torch.equal(got[0][:, :9], batch)
    with pytest.raises(ValueError):
        decoder.generate(batch, 4, eos_token_id=1)


from bench import FLUX_PATTERNS, FluxShapedDiT          # the benchmark's FLUX-shaped stack, here at toy size


def _TinyDiT():
    return FluxShapedDiT(h=128, heads=4, n_double=2, n_single=2)


@pytest.mark.gpu
@pytest.mark.parametrize("offload", [False, True])
def test_diffusion_transformer_with_the_flux_pattern_dictionary(tmp_path, offload):
    """Units of 14 and 6 Linear layers with biases, named through dotted paths (ModuleList
    indices included): single-file save, load, one forward = the BF16 model's, bit for bit."""
    torch.manual_seed(21)
    net = _TinyDiT().to(torch.bfloat16).eval()
    with torch.no_grad():
        for p in net.parameters():
            p.copy_((torch.randn(p.shape) * 0.05).to(torch.bfloat16))
    reference = copy.deepcopy(net).to("cuda:0")
    path = str(tmp_path / "dit")
    df11.compress_model(net, FLUX_PATTERNS, path, save_single_file=True, check_correctness=True)
    torch.manual_seed(22)
    skeleton = _TinyDiT().to(torch.bfloat16).eval()
    model = df11.DFloat11Model.from_single_file(os.path.join(path, "model.safetensors"), pattern_dict=FLUX_PATTERNS,
                                                bfloat16_model=skeleton, device="cuda:0", cpu_offload=offload)
    g = torch.Generator().manual_seed(23)
    x = torch.randn(2, 24, 128, generator=g).to(torch.bfloat16).to("cuda:0")
    ctx = torch.randn(2, 7, 128, generator=g).to(torch.bfloat16).to("cuda:0")
    cond = torch.randn(2, 1, 128, generator=g).to(torch.bfloat16).to("cuda:0")
    with torch.no_grad():
        for _ in range(2):
            assert torch.equal(model(x, ctx, cond), reference(x, ctx, cond))
    assert len(model.transformer_blocks[0].weight_injection_modules) == 14
    assert not isinstance(model.transformer_blocks[1].attn.to_out[0].weight, nn.Parameter)   # an injected view


def test_mapped_safetensors_reader_round_trips_every_dtype(tmp_path):
    """`safetensors_io.MappedFile` against `safetensors.torch.save_file` / `load_file`: names in
    file order, shapes, dtypes (BF16 included, which numpy does not know) and bytes; a tensor
    taken out owns its memory; malformed files are refused."""
    from safetensors.torch import load_file, save_file
    from dfloat11_b200.safetensors_io import MappedFile
    g = torch.Generator().manual_seed(0)
    tensors = {
        "a.bf16": torch.randn(33, 7, generator=g).to(torch.bfloat16),
        "b.u8": torch.randint(0, 256, (1000,), generator=g, dtype=torch.uint8),
        "c.f32": torch.randn(5, generator=g),
        "d.i64": torch.arange(12).view(3, 4),
        "e.f16": torch.randn(2, 2, 2, generator=g).to(torch.float16),
        "f.empty": torch.zeros(0, dtype=torch.uint8),
    }
    path = str(tmp_path / "t.safetensors")
    save_file(tensors, path)
    want = load_file(path)
    with MappedFile(path) as mapped:
        assert set(mapped.names()) == set(tensors)
        for name in mapped.names():
            got = mapped.tensor(name)
            assert got.dtype == want[name].dtype and got.shape == want[name].shape
            assert torch.equal(got.view(torch.uint8), want[name].view(torch.uint8) if want[name].numel() else got.view(torch.uint8))
            assert mapped.nbytes(name) == want[name].numel() * want[name].element_size()
        kept = mapped.tensor("a.bf16")
    assert torch.equal(kept, tensors["a.bf16"])                  # still valid after the mapping is closed
    for bad in (b"", b"\x10\x00\x00\x00\x00\x00\x00\x00{}", (10 ** 6).to_bytes(8, "little") + b"{}"):
        broken = str(tmp_path / "broken.safetensors")
        with open(broken, "wb") as f:
            f.write(bad)
        with pytest.raises((ValueError, OSError)):
            MappedFile(broken)
