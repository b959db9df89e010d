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
  * store_*.npz    : the Triton kernel `store_kvcache` (interpreter).
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
REF = os.environ.get("MINIVLLM_REFERENCE", os.path.join(os.sep, "root", "reference"))
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


if __name__ == "__main__":
    only = [a for a in sys.argv[1:] if a.startswith("--only=")]
    which = only[0].split("=")[1].split(",") if only else ["ops", "metadata", "prenorm"]
    if "ops" in which:
        main()
    if "metadata" in which:
        metadata_main()
    if "prenorm" in which:
        prenorm_main()
