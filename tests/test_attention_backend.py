"""The compressed-prefix attention function inside a Hugging Face model.

CPU: the host logic (cache layer lengths, positions, tensor layouts, log-sum-exp merge of
prefix and tail) with a stand-in for the kernel library that attends over an fp16 copy of the
prefix -- logits must match the model's own attention over the same cache.
GPU: the real library over turbo_mse pages written by ``CAGStore.pack_document`` -- logits must
match the reference's flow (dequantise the stored document into a ``DynamicCache``, run the
model's own attention) within the tolerance the attention kernels are held to.
"""
import math

import pytest

torch = pytest.importorskip("torch")
transformers = pytest.importorskip("transformers")

from turborag_b200 import attention_backend as ab  # noqa: E402


def tiny_model(dtype, device):
    from transformers import Qwen2Config, Qwen2ForCausalLM
    torch.manual_seed(7)
    cfg = Qwen2Config(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=4096,
                      attn_implementation="eager")
    model = Qwen2ForCausalLM(cfg).to(dtype).to(device).eval()
    assert model.model.layers[0].self_attn.head_dim == 128
    return model


def layer_kv(past, layer):
    lyr = past.layers[layer]
    return lyr.keys, lyr.values


class TorchStandIn:
    """Stand-in for the kernel library on machines without a GPU: same methods and record
    format the attention function uses, arithmetic in torch over an fp16 prefix."""

    class _Cfg:
        num_kv_heads, head_dim, block_size = 2, 128, 16

    def __init__(self, prefix):  # prefix: {id(pool) -> (k [H, N, D], v [H, N, D])}
        self.prefix = prefix

    def mse_prefill_paged(self, q, pool, tables, lens, ck, cv, out, layout, cfg, stream=0):
        k0, v0 = self.prefix[id(pool)]
        _, sq, hq, d = q.shape
        g = hq // k0.shape[0]
        k = torch.cat([k0, ck[0].transpose(0, 1)], dim=1).float().repeat_interleave(g, 0)
        v = torch.cat([v0, cv[0].transpose(0, 1)], dim=1).float().repeat_interleave(g, 0)
        s = torch.matmul(q[0].transpose(0, 1).float(), k.transpose(1, 2)) / math.sqrt(d)
        n = k0.shape[1]
        causal = torch.arange(sq).view(-1, 1) + n >= torch.arange(n + sq).view(1, -1)
        s = s.masked_fill(~causal, float("-inf"))
        out.copy_(torch.matmul(torch.softmax(s, -1), v).transpose(0, 1).unsqueeze(0).to(out.dtype))

    def decode_paged(self, scheme, q, pool, tables, lens, layout, cfg, partials_out=None, stream=0):
        k0, v0 = self.prefix[id(pool)]
        hq, d = q.shape[1], q.shape[2]
        g = hq // k0.shape[0]
        s = torch.einsum("hd,hnd->hn", q[0].float(), k0.float().repeat_interleave(g, 0)) / math.sqrt(d)
        m = s.max(-1).values
        p = torch.exp(s - m.unsqueeze(-1))
        partials_out[0, :, :128] = torch.einsum("hn,hnd->hd", p, v0.float().repeat_interleave(g, 0))
        partials_out[0, :, 128] = m
        partials_out[0, :, 129] = p.sum(-1)

    def merge_partials(self, partials, output, hq, hkv, stream=0):
        output.copy_((partials[0, :, :128] / partials[0, :, 129:130]).to(output.dtype))


def run_question(model, cache, question, steps):
    """Question chunk, then ``steps`` greedy tokens; returns the logits of every forward."""
    logits = []
    with torch.no_grad():
        out = model(question, past_key_values=cache, use_cache=True)
        logits.append(out.logits[0, -1].float())
        for _ in range(steps):
            nxt = logits[-1].argmax().view(1, 1)
            out = model(nxt, past_key_values=cache, use_cache=True)
            logits.append(out.logits[0, -1].float())
    return logits


def generate_like_reference(model, cache, question, n_prefix, steps):
    """The call the reference's runner makes (tq_backend/benchmark.py:250-262): question tokens only,
    positions continuing after the document, attention mask over document + question."""
    q_len = question.shape[1]
    pos = torch.arange(n_prefix, n_prefix + q_len, device=question.device).unsqueeze(0)
    mask = torch.ones(1, n_prefix + q_len, device=question.device, dtype=torch.long)
    with torch.no_grad():
        out = model.generate(input_ids=question, attention_mask=mask, past_key_values=cache, position_ids=pos,
                             max_new_tokens=steps, do_sample=False, temperature=None, top_p=None)
    return out[0, q_len:].tolist()


def test_cache_layer_reports_prefix_plus_tail():
    cache = ab.compressed_prefix_cache(300, 2)
    assert cache.get_seq_length() == 300
    k = torch.zeros(1, 2, 5, 128)
    rk, rv = cache.update(k, k, 0)
    assert rk.shape[2] == 5 and cache.get_seq_length(0) == 305
    rk, _ = cache.update(k[:, :, :1], k[:, :, :1], 0)
    assert rk.shape[2] == 6 and cache.get_seq_length(0) == 306


def test_host_logic_matches_model_attention_cpu():
    model = tiny_model(torch.float32, "cpu")
    g = torch.Generator().manual_seed(3)
    doc = torch.randint(0, 512, (1, 77), generator=g)
    question = torch.randint(0, 512, (1, 9), generator=g)
    with torch.no_grad():
        past = model(doc, use_cache=True).past_key_values
    ref = run_question(model, past, question, steps=3)
    with torch.no_grad():
        past = model(doc, use_cache=True).past_key_values
    ref_tokens = generate_like_reference(model, past, question, 77, steps=5)

    with torch.no_grad():
        past = model(doc, use_cache=True).past_key_values
    prefix, pools = {}, []
    for l in range(2):
        k, v = layer_kv(past, l)
        pool = torch.zeros(1)
        pools.append(pool)
        prefix[id(pool)] = (k[0].clone(), v[0].clone())
    ab.register()
    rt = ab._Runtime(TorchStandIn(prefix), TorchStandIn._Cfg, None)
    for m, pool in zip(ab._attention_modules(model), pools):
        m._tq_prefix = ab.LayerPrefix(pool, 77, torch.zeros(1, 5, dtype=torch.int32), torch.tensor([77]))
        m._tq_runtime = rt
    model.config._attn_implementation = ab.ATTENTION_NAME
    # the function insists on fp16 and a CUDA stream; lift both checks for the stand-in run
    real = ab.turborag_mse_attention

    def on_cpu(module, query, key, value, *a, **kw):
        class _S:
            cuda_stream = 0
        orig = torch.cuda.current_stream
        torch.cuda.current_stream = lambda *_: _S
        try:
            o, _ = real(module, query.half(), key, value, *a, **kw)
        finally:
            torch.cuda.current_stream = orig
        return o.float(), None

    from transformers import AttentionInterface
    AttentionInterface.register(ab.ATTENTION_NAME, on_cpu)
    try:
        got = run_question(model, ab.compressed_prefix_cache(77, 2), question, steps=3)
        got_tokens = generate_like_reference(model, ab.compressed_prefix_cache(77, 2), question, 77, steps=5)
        # the question in two chunks: the second one meets an older fp16 tail
        cache2 = ab.compressed_prefix_cache(77, 2)
        with torch.no_grad():
            model(question[:, :5], past_key_values=cache2, use_cache=True)
            two_chunks = model(question[:, 5:], past_key_values=cache2, use_cache=True).logits[0, -1].float()
    finally:
        AttentionInterface.register(ab.ATTENTION_NAME, real)
        ab.uninstall(model)
    for r, o in zip(ref, got):
        assert (r - o).abs().max() < 2e-2 * r.abs().max()
        assert r.argmax() == o.argmax()
    assert got_tokens == ref_tokens and len(ref_tokens) == 5  # model.generate drives the cache layer too
    assert (two_chunks - ref[0]).abs().max() < 2e-2 * ref[0].abs().max()


def test_unattached_layer_raises():
    with pytest.raises(RuntimeError):
        ab.turborag_mse_attention(torch.nn.Identity(), torch.zeros(1, 4, 1, 128), None, None)


@pytest.mark.gpu
@pytest.mark.parametrize("scheme", ["turbo_mse", "turbo_prod"])
def test_model_logits_match_dequantised_cache(tmp_path, scheme):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from turborag_b200.store import CAGStore
    dev = torch.device("cuda:0")
    model = tiny_model(torch.float16, dev)
    g = torch.Generator().manual_seed(11)
    doc = torch.randint(0, 512, (1, 300), generator=g).to(dev)
    question = torch.randint(0, 512, (1, 21), generator=g).to(dev)
    store = CAGStore(tmp_path)
    with torch.no_grad():
        past = model(doc, use_cache=True).past_key_values
    for l in range(2):
        k, v = layer_kv(past, l)
        store.pack_document("doc", l, k[0].permute(1, 0, 2).contiguous(), v[0].permute(1, 0, 2).contiguous(),
                            scheme)
    # the reference's flow: stored pages -> fp16 DynamicCache -> the model's own attention
    cache, n = store.build_dynamic_cache("doc", 2, scheme, (2, 128))
    assert n == 300
    ref = run_question(model, cache, question, steps=4)
    cache, _ = store.build_dynamic_cache("doc", 2, scheme, (2, 128))
    ref_tokens = generate_like_reference(model, cache, question, 300, steps=6)
    # this module: the pages stay compressed
    cache, n2 = store.attach_to_model(model, "doc", 2, (2, 128), scheme)
    assert n2 == 300
    try:
        got = run_question(model, cache, question, steps=4)
        got_tokens = generate_like_reference(model, ab.compressed_prefix_cache(300, 2), question, 300, steps=6)
    finally:
        ab.uninstall(model)
    assert store.tq.mse_prefill_status() == 0
    assert got_tokens == ref_tokens, (got_tokens, ref_tokens)
    # the same document from the one-file container
    store.export_container("doc", 2, scheme, (2, 128))
    cache, _ = store.attach_to_model(model, "doc", 2, (2, 128), scheme)
    try:
        again = run_question(model, cache, question, steps=1)
    finally:
        ab.uninstall(model)
    assert torch.equal(again[0], got[0]) and torch.equal(again[1], got[1])
    for r, o in zip(ref, got):
        assert (r - o).abs().max() < 2e-2 * r.abs().max(), (r - o).abs().max() / r.abs().max()
