"""Generates tests/golden/*.npz by running the REFERENCE's own code on the CPU.

Run once, where a checkout of the reference is at hand; its location comes from
$MINIVLLM_REFERENCE:

    MINIVLLM_REFERENCE=<reference checkout> python tests/golden/make_golden.py

What is recorded (inputs are regenerated from seeds by the tests; only the
reference's outputs are stored, as fp32):
  * decode_*.npz   : benchmark_decoding.py `decode_torch_optimized` and
                     `naive_decode_attention`, and the Triton kernel
                     `paged_attention_decode` under TRITON_INTERPRET=1;
  * prefill_*.npz  : benchmark_prefilling.py `pytorch_standard_attention` and
                     the Triton kernel `flash_attention_prefill` (interpreter);
  * store_*.npz    : the Triton kernel `store_kvcache` (interpreter);
  * layers_small.npz : the reference's LayerNorm (residual add + RMSNorm) and SiluAndMul modules;
  * model_logits.npz : the reference's whole Qwen3ForCausalLM (models/qwen3.py), fp32, toy size, with the
                     harness model's seeded weights copied in: logits of one prefill and one decode step.
The fixtures are small so that the interpreter finishes in seconds and the
files stay a few hundred KB.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("MINIVLLM_REFERENCE")
if not REF or not os.path.isdir(REF):
    sys.exit("set MINIVLLM_REFERENCE to a checkout of the reference engine")
sys.path.insert(0, ROOT)
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "src"))

from minivllm_b200 import synth  # noqa: E402

# Cases: name -> generator kwargs.  Rounded to fp16/bf16 first, then fed to the reference in fp32.
DECODE_CASES = {
    "decode_small_bs16": dict(seed=10, batch=3, ctx_lo=5, ctx_hi=70, num_heads=4, num_kv_heads=2, head_dim=64,
                              block_size=16),
    "decode_gqa4_bs256": dict(seed=11, batch=4, ctx_lo=64, ctx_hi=600, num_heads=8, num_kv_heads=2, head_dim=128,
                              block_size=256),
    "decode_cfg0_like": dict(seed=0, batch=16, ctx_lo=64, ctx_hi=1024, num_heads=16, num_kv_heads=8, head_dim=128,
                             block_size=256),
}
PREFILL_CASES = {
    "prefill_small": dict(seed=20, num_seqs=3, len_lo=1, len_hi=70, num_heads=4, num_kv_heads=2, head_dim=64),
    "prefill_gqa4": dict(seed=21, num_seqs=3, len_lo=40, len_hi=200, num_heads=8, num_kv_heads=2, head_dim=128),
}
STORE_CASES = {
    "store_small": dict(seed=30, num_tokens=40, num_blocks=8, block_size=16, num_kv_heads=2, head_dim=64,
                        pad_frac=0.2),
}
TRITON_MAX_TOKENS = 3000  # interpreter budget


def rounded(x, dtype):
    return x.to(dtype).to(torch.float32)


def main():
    import benchmark_decoding as bd
    import benchmark_prefilling as bp
    from myvllm.layers import attention as ref_attn

    for name, kw in DECODE_CASES.items():
        d = synth.decode_inputs(**kw)
        q, kc, vc = (rounded(d[k], torch.float16) for k in ("q", "k_cache", "v_cache"))
        args = (q, kc, vc, d["block_tables"], d["context_lens"], d["scale"], d["num_heads"], d["num_kv_heads"],
                d["head_dim"], d["block_size"])
        out = {"torch_optimized": bd.decode_torch_optimized(*args).numpy(),
               "naive": bd.naive_decode_attention(*args).numpy()}
        if int(d["context_lens"].sum()) <= TRITON_MAX_TOKENS:
            out["triton"] = ref_attn.paged_attention_decode(*args).numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), kwargs=repr(kw), **out)
        print(name, {k: v.shape for k, v in out.items()})

    for name, kw in PREFILL_CASES.items():
        d = synth.prefill_inputs(**kw)
        q, k, v = (rounded(d[x], torch.bfloat16) for x in ("q", "k", "v"))
        args = (q, k, v, d["cu_seqlens"], d["scale"], d["num_heads"], d["num_kv_heads"], d["head_dim"])
        out = {"torch_standard": bp.pytorch_standard_attention(*args).numpy()}
        if q.shape[0] <= TRITON_MAX_TOKENS:
            out["triton"] = ref_attn.flash_attention_prefill(*args).numpy()
        np.savez_compressed(os.path.join(HERE, name + ".npz"), kwargs=repr(kw), **out)
        print(name, {k: v.shape for k, v in out.items()})

    for name, kw in STORE_CASES.items():
        d = synth.store_inputs(**kw)
        k, v = rounded(d["k"], torch.bfloat16), rounded(d["v"], torch.bfloat16)
        shape = (d["num_blocks"], d["block_size"], d["num_kv_heads"], d["head_dim"])
        kc = torch.full(shape, -7.0)
        vc = torch.full(shape, -7.0)
        ref_attn.store_kvcache(k, v, kc, vc, d["slot_mapping"], d["block_size"])
        np.savez_compressed(os.path.join(HERE, name + ".npz"), kwargs=repr(kw), k_cache=kc.numpy(), v_cache=vc.numpy())
        print(name, kc.shape)




# ---------------------------------------------------------------------------
# Step metadata: the reference's Sequence / BlockManager / ModelRunner.prepare_*
# run on the CPU (torch.tensor(pin_memory=...) and Tensor.cuda are shimmed).
# ---------------------------------------------------------------------------
METADATA_CASES = {
    # block_size, prompts (token id lists), tokens appended afterwards (one decode step each)
    "metadata_bs4": dict(block_size=4, prompts=[list(range(1, 11)), list(range(1, 9)) + [42], [7, 7, 7]],
                         appended=[[11], [12], [13]]),
    "metadata_bs16": dict(block_size=16, prompts=[list(range(100, 137)), list(range(5)), list(range(300, 331))],
                          appended=[[1, 2], [3, 4], [5, 6]]),
}


def metadata_main():
    import types
    from myvllm.engine import model_runner as mr
    from myvllm.engine.block_manager import BlockManager
    from myvllm.engine.sequence import Sequence
    from myvllm.utils.context import get_context

    real_tensor = torch.tensor
    mr.torch.tensor = lambda *a, **k: real_tensor(*a, **{x: y for x, y in k.items() if x != "pin_memory"})
    torch.Tensor.cuda = lambda self, *a, **k: self
    try:
        for name, case in METADATA_CASES.items():
            bs = case["block_size"]
            Sequence.block_size = bs
            bm = BlockManager(64, bs)
            seqs = [Sequence(token_ids=list(p)) for p in case["prompts"]]
            for s in seqs:
                bm.allocate(s)
            stub = types.SimpleNamespace(block_size=bs)
            out = {}
            ids = mr.ModelRunner.prepare_prefill(stub, seqs)
            c = get_context()
            out.update(prefill_input_ids=ids.numpy(), prefill_cu_q=c.cu_seqlens_q.numpy(),
                       prefill_cu_k=c.cu_seqlens_k.numpy(), prefill_slot_mapping=c.slot_mapping.numpy(),
                       prefill_num_cached=np.array([s.num_cached_tokens for s in seqs]),
                       prefill_tables=np.array([s.block_table + [-1] * (8 - len(s.block_table)) for s in seqs]))
            steps = len(case["appended"][0])
            for t in range(steps):
                for s, extra in zip(seqs, case["appended"]):
                    s.append_token(extra[t])      # the intended postprocess (the reference appends to token_ids only)
                    bm.append(s) if bm.can_append(s) else None
                ids = mr.ModelRunner.prepare_decode(stub, seqs)
                c = get_context()
                out[f"decode{t}_input_ids"] = ids.numpy()
                out[f"decode{t}_context_lens"] = c.context_lens.numpy()
                out[f"decode{t}_slot_mapping"] = c.slot_mapping.numpy()
                out[f"decode{t}_block_tables"] = c.block_tables.numpy()
                out[f"decode{t}_tables_full"] = np.array([s.block_table + [-1] * (8 - len(s.block_table)) for s in seqs])
            np.savez_compressed(os.path.join(HERE, name + ".npz"), case=repr(case), **out)
            print(name, sorted(out))
    finally:
        mr.torch.tensor = real_tensor




def prenorm_main():
    """q/k RMSNorm + rotary embedding through the reference's own LayerNorm and RotaryEmbedding (fp32, CPU)."""
    from myvllm.layers.layernorm import LayerNorm
    from myvllm.layers.rotary_embedding import RotaryEmbedding
    g = torch.Generator().manual_seed(40)
    tokens, heads, kv_heads, d = 37, 4, 2, 128
    q = torch.randn(tokens, heads, d, generator=g)
    k = torch.randn(tokens, kv_heads, d, generator=g) * 3
    gamma = torch.rand(d, generator=g) + 0.5
    positions = torch.randint(0, 500, (tokens,), generator=g)
    norm = LayerNorm(gamma)                      # eps defaults to 1e-5, as in the engine
    rope = RotaryEmbedding(base=1000000, rotary_embedding=d, max_position=512)
    qo, ko = rope(positions, norm(q), norm(k))
    np.savez_compressed(os.path.join(HERE, "prenorm_rope.npz"), q=qo.numpy(), k=ko.numpy(), seed=40,
                        shape=np.array([tokens, heads, kv_heads, d]))
    print("prenorm_rope", qo.shape, ko.shape)


def layers_main():
    """Residual add + RMSNorm and the SwiGLU activation through the reference's own modules (fp32, CPU):
    LayerNorm.forward(x, residual) (src/myvllm/layers/layernorm.py:24-28) and SiluAndMul
    (src/myvllm/layers/activation.py:17-20)."""
    from myvllm.layers.activation import SiluAndMul
    from myvllm.layers.layernorm import LayerNorm
    g = torch.Generator().manual_seed(50)
    x = torch.randn(11, 96, generator=g)
    residual = torch.randn(11, 96, generator=g) * 2
    gamma = torch.rand(96, generator=g) + 0.5
    normed, new_res = LayerNorm(gamma)(x, residual)
    plain = LayerNorm(gamma)(x)
    gu = torch.randn(7, 2 * 40, generator=g) * 2
    act = SiluAndMul()(gu)
    np.savez_compressed(os.path.join(HERE, "layers_small.npz"), seed=50, normed=normed.numpy(),
                        new_residual=new_res.numpy(), plain=plain.numpy(), act=act.numpy())
    print("layers_small", normed.shape, act.shape)


MODEL_CASE = dict(vocab_size=211, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                  intermediate_size=96, max_position=64, block_size=16, seed=3, lens=(5, 9))


def model_main():
    """Logits of the reference's own Qwen3ForCausalLM (src/myvllm/models/qwen3.py:276-331) on the CPU in fp32:
    one prefill step over two sequences and one decode step, attention through the reference's Triton kernels
    (interpreter).  The weights are the harness model's seeded weights copied in; the only shims are the ones
    the reference cannot run without: a one-rank gloo group (its layers query the process group), biases off,
    `Attention.block_size` set to the cache's block size, and the context set by hand as its model runner
    would (src/myvllm/engine/model_runner.py:217-226,246-255)."""
    import torch.distributed as dist
    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29779", world_size=1, rank=0)
    from myvllm.models.qwen3 import Qwen3ForCausalLM as RefModel
    from myvllm.utils import reset_context, set_context
    from minivllm_b200.engine.qwen3 import Qwen3Config, Qwen3ForCausalLM
    c = MODEL_CASE
    cfg = Qwen3Config(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_layers=c["num_layers"],
                      num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"], head_dim=c["head_dim"],
                      intermediate_size=c["intermediate_size"], max_position=c["max_position"],
                      block_size=c["block_size"], tie_word_embeddings=True)
    ours = Qwen3ForCausalLM(cfg, 0, 1, torch.float32, "cpu", seed=c["seed"])
    ref = RefModel(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_heads=c["num_heads"],
                   head_dim=c["head_dim"], num_kv_heads=c["num_kv_heads"], intermediate_size=c["intermediate_size"],
                   num_layers=c["num_layers"], base=1000000, max_position=c["max_position"], ffn_bias=False,
                   qkv_bias=False, tie_word_embeddings=True)
    with torch.no_grad():
        ref.qwen3_model.embedding_layer.weight.copy_(ours.embed)
        for mine, theirs in zip(ours.layers, ref.qwen3_model.layer_stack):
            theirs.self_attn.qkv_projection.weight.copy_(mine.qkv_w)
            theirs.self_attn.output_projection.weight.copy_(mine.o_w)
            theirs.mlp.gate_up.weight.copy_(mine.gate_up_w)
            theirs.mlp.gate_down.weight.copy_(mine.down_w)
    bs, lens = c["block_size"], c["lens"]
    kv = torch.zeros(2, c["num_layers"], 4, bs, c["num_kv_heads"], c["head_dim"])
    for l, layer in enumerate(ref.qwen3_model.layer_stack):
        a = layer.self_attn.attention
        a.k_cache, a.v_cache, a.block_size = kv[0, l], kv[1, l], bs
    g = torch.Generator().manual_seed(c["seed"])
    ids = torch.randint(0, c["vocab_size"], (sum(lens),), generator=g)
    cu = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32)
    tables = torch.tensor([[2], [0]], dtype=torch.int32)             # one 16-token block per sequence
    slot_prefill = torch.cat([tables[i, 0].long() * bs + torch.arange(n) for i, n in enumerate(lens)])
    with torch.inference_mode():
        set_context(True, cu, cu, max(lens), max(lens), slot_prefill, None, None)
        prefill_logits = ref.compute_logits(ref(ids)).clone()
        tok = prefill_logits.argmax(-1)
        ctx_lens = torch.tensor([n + 1 for n in lens], dtype=torch.int32)
        slot_decode = torch.tensor([int(tables[i, 0]) * bs + n for i, n in enumerate(lens)], dtype=torch.int64)
        set_context(False, None, None, 0, 0, slot_decode, ctx_lens, tables)
        decode_logits = ref.compute_logits(ref(tok)).clone()
        reset_context()
    np.savez_compressed(os.path.join(HERE, "model_logits.npz"), case=repr(c), input_ids=ids.numpy(),
                        prefill_logits=prefill_logits.numpy(), decode_input=tok.numpy(),
                        decode_logits=decode_logits.numpy())
    print("model_logits", prefill_logits.shape, decode_logits.shape, tok.tolist())


if __name__ == "__main__":
    only = [a for a in sys.argv[1:] if a.startswith("--only=")]
    which = only[0].split("=")[1].split(",") if only else ["ops", "metadata", "prenorm", "layers", "model"]
    if "ops" in which:
        main()
    if "metadata" in which:
        metadata_main()
    if "prenorm" in which:
        prenorm_main()
    if "layers" in which:
        layers_main()
    if "model" in which:
        model_main()
