"""The vLLM-facing hook checked without a GPU: op registration under the reference's names and
schemas (mutated buffer, fake implementation), the plugin entry point, CustomOp subclassing against
the installed vLLM, and the constructor / forward signatures."""
import inspect
import os

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _ns():
    from transarch_b200 import vllm_hook
    return getattr(torch.ops, vllm_hook.OP_NAMESPACE)


def test_register_defines_ops_with_fake_impl():
    from transarch_b200 import vllm_hook
    vllm_hook.register()
    vllm_hook.register()                                   # idempotent
    if vllm_hook.HAVE_VLLM:
        assert vllm_hook.OP_NAMESPACE == "vllm"            # where the reference registers (indexers.py:607-613)
    op = _ns().misa_sparse_attn_indexer
    schema = op.default._schema
    names = [a.name for a in schema.arguments]
    assert names == ["hidden_states", "k_cache_prefix", "kv_cache", "q_fp8", "k", "weights", "q_head_topk_indices",
                     "quant_block_size", "scale_fmt", "topk_heads", "decode_topk_heads", "use_qnorm",
                     "k_block_size", "stage1_topk", "topk_tokens", "head_dim", "max_model_len", "total_seq_lens",
                     "topk_indices_buffer"]
    assert schema.arguments[-1].alias_info is not None and schema.arguments[-1].alias_info.is_write
    assert all(a.alias_info is None for a in schema.arguments[:-1])       # nothing else is mutated
    base = _ns().baseline_sparse_attn_indexer.default._schema
    assert [a.name for a in base.arguments] == [
        "hidden_states", "k_cache_prefix", "kv_cache", "q_fp8", "k", "weights", "quant_block_size", "scale_fmt",
        "topk_tokens", "head_dim", "max_model_len", "total_seq_lens", "topk_indices_buffer"]
    assert base.arguments[-1].alias_info.is_write
    T = 5
    m = lambda *s, dt=torch.bfloat16: torch.empty(*s, dtype=dt, device="meta")
    buf = m(T, 2048, dt=torch.int32)
    out = op(m(T, 7168), "model.layers.0.self_attn.indexer.k_cache", m(4, 64, 132, dt=torch.uint8),
             m(T, 64, 128, dt=torch.float8_e4m3fn), m(T, 128), m(T, 64, dt=torch.float32), None, 128, "ue8m0",
             8, 8, False, 1024, 8192, 2048, 128, 65536, 0, buf)
    assert out.shape == buf.shape and out.dtype == torch.int32 and out.device.type == "meta"


def test_plugin_entry_point_resolves_to_register():
    import importlib
    import tomllib
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        proj = tomllib.load(f)
    eps = proj["project"]["entry-points"]["vllm.general_plugins"]
    assert len(eps) == 1
    target = next(iter(eps.values()))
    mod, fn = target.split(":")
    obj = getattr(importlib.import_module(mod), fn)
    from transarch_b200 import vllm_hook
    assert obj is vllm_hook.register


def test_custom_op_classes_against_installed_vllm():
    from transarch_b200 import vllm_hook
    if not vllm_hook.HAVE_VLLM:
        pytest.skip("vLLM is not importable here")
    from vllm.model_executor.custom_op import CustomOp, op_registry
    vllm_hook.register()
    assert issubclass(vllm_hook.MiSASparseAttnIndexer, CustomOp)
    assert issubclass(vllm_hook.BaselineSparseAttnIndexer, CustomOp)
    assert op_registry["misa_sparse_attn_indexer"] is vllm_hook.MiSASparseAttnIndexer
    assert op_registry["baseline_sparse_attn_indexer"] is vllm_hook.BaselineSparseAttnIndexer
    buf = torch.zeros(4, 16, dtype=torch.int32)
    cache = torch.zeros(2, 64, 132, dtype=torch.uint8)
    op = vllm_hook.MiSASparseAttnIndexer(cache, 128, "ue8m0", 8, 8, True, 1024, 8192, 2048, 128, 4096, 8192, buf)
    assert op.topk_tokens == 2048 and op.scale_fmt == "ue8m0" and isinstance(op, torch.nn.Module)
    base = vllm_hook.BaselineSparseAttnIndexer(cache, 128, "ue8m0", 2048, 128, 4096, 8192, buf)
    assert base.use_misa is False
    # the adapter takes the constructor of the installed vLLM's own layer
    from vllm.model_executor.layers.sparse_attn_indexer import SparseAttnIndexer
    want = list(inspect.signature(SparseAttnIndexer.__init__).parameters)
    got = list(inspect.signature(vllm_hook.SparseAttnIndexer022.__init__).parameters)
    assert got == want
    want_f = list(inspect.signature(SparseAttnIndexer.forward_cuda).parameters)
    got_f = list(inspect.signature(vllm_hook.SparseAttnIndexer022.forward_cuda).parameters)
    assert got_f[:len(want_f)] == want_f
    ad = vllm_hook.SparseAttnIndexer022(cache, 128, "ue8m0", 2048, 128, 4096, 8192, buf, skip_k_cache_insert=True)
    assert ad.skip_k_cache_insert is True
    # a profiling / dummy run (no metadata in scope) leaves the buffer untouched and returns it
    out = ad.forward_cuda(torch.zeros(4, 8), torch.zeros(4, 64, 128), torch.zeros(4, 128), torch.zeros(4, 64))
    assert out is buf


def test_hook_classes_mirror_reference_constructor():
    from transarch_b200 import vllm_hook
    params = list(inspect.signature(vllm_hook.MiSASparseAttnIndexer.__init__).parameters)[1:]
    assert params == ["k_cache", "quant_block_size", "scale_fmt", "topk_heads", "decode_topk_heads", "use_qnorm",
                      "k_block_size", "stage1_topk", "topk_tokens", "head_dim", "max_model_len",
                      "max_total_seq_len", "topk_indices_buffer"]
    # the reference's positional arguments first; anything after them (the metadata a caller may
    # pass when there is no vLLM forward context) must be optional
    sig = inspect.signature(vllm_hook.MiSASparseAttnIndexer.forward_cuda).parameters
    fwd = list(sig)[1:]
    assert fwd[:5] == ["hidden_states", "q_fp8", "k", "weights", "q_head_topk_indices"]
    assert all(sig[n].default is not inspect.Parameter.empty for n in fwd[5:])
    base = list(inspect.signature(vllm_hook.BaselineSparseAttnIndexer.__init__).parameters)[1:]
    assert base == ["k_cache", "quant_block_size", "scale_fmt", "topk_tokens", "head_dim", "max_model_len",
                    "max_total_seq_len", "topk_indices_buffer"]


def test_decode_row_contexts_uniform_padded_and_per_row():
    """Keys visible to each decode token: uniform next_n, the padded (mixed decode lengths) layout of
    the reference (indexers.py:165-171, :521-551) and vLLM 0.22's per-row [B, next_n] lengths."""
    from transarch_b200.vllm_hook import DecodeMetadata, _decode_rows
    seq = torch.tensor([100, 50, 7], dtype=torch.int32)
    tbl = torch.zeros(3, 4, dtype=torch.int32)
    ctx, rt, nn = _decode_rows(DecodeMetadata(seq, tbl), 6)
    assert nn == 2 and rt is None and ctx.tolist() == [99, 100, 49, 50, 6, 7]
    # padded: decode_lens 2, 1, 2 -> reference pads to next_n = 2; request 1's only token sits in padded slot 0
    dm = DecodeMetadata(seq, tbl, decode_lens=torch.tensor([2, 1, 2]), requires_padding=True)
    ctx, rt, nn = _decode_rows(dm, 5)
    assert nn == 1 and rt.tolist() == [0, 0, 1, 2, 2] and ctx.tolist() == [99, 100, 49, 6, 7]
    per_row = torch.tensor([[99, 100], [49, 50], [6, 7]], dtype=torch.int32)
    ctx, rt, nn = _decode_rows(DecodeMetadata(per_row, tbl), 6)
    assert nn == 2 and rt is None and ctx.tolist() == [99, 100, 49, 50, 6, 7]
