"""The harness model (minivllm_b200/engine/qwen3.py) against the REFERENCE's own Qwen3ForCausalLM: logits of one
prefill step and one decode step, fp32 on the CPU, attention through the CPU oracle on our side and through the
reference's Triton kernels on theirs (recorded by tests/golden/make_golden.py --only=model with the same seeded
weights).  This pins the layer arithmetic around the attention path -- shared q/k gamma, eps 1e-5, rotate-half
RoPE, head split, SwiGLU, tied head, and the residual stream that starts from the normalised embedding -- to the
reference model itself."""
import ast
import os

import numpy as np
import torch

from minivllm_b200.engine.qwen3 import Qwen3Config, Qwen3ForCausalLM
from minivllm_b200.utils.context import reset_context, set_context
from oracle.attention_module import swap_in_oracle_attention

HERE = os.path.dirname(os.path.abspath(__file__))


def test_prefill_and_decode_logits_match_the_reference_model():
    z = np.load(os.path.join(HERE, "golden", "model_logits.npz"))
    c = ast.literal_eval(str(z["case"]))
    cfg = Qwen3Config(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_layers=c["num_layers"],
                      num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"], head_dim=c["head_dim"],
                      intermediate_size=c["intermediate_size"], max_position=c["max_position"],
                      block_size=c["block_size"], tie_word_embeddings=True)
    model = swap_in_oracle_attention(Qwen3ForCausalLM(cfg, 0, 1, torch.float32, "cpu", seed=c["seed"]))
    bs, lens = c["block_size"], c["lens"]
    kv = torch.zeros(2, c["num_layers"], 4, bs, c["num_kv_heads"], c["head_dim"])
    for l, layer in enumerate(model.layers):
        layer.attn.k_cache, layer.attn.v_cache = kv[0, l], kv[1, l]
    ids = torch.from_numpy(z["input_ids"])
    cu = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32)
    tables = torch.tensor([[2], [0]], dtype=torch.int32)
    slots = torch.cat([tables[i, 0].long() * bs + torch.arange(n) for i, n in enumerate(lens)])
    with torch.inference_mode():
        set_context(True, cu, cu, max(lens), max(lens), slots, None, None,
                    positions=torch.cat([torch.arange(n) for n in lens]), last_token_index=(cu[1:] - 1).long())
        prefill = model.compute_logits(model(ids))
        tok = prefill.argmax(-1)
        assert tok.tolist() == z["decode_input"].tolist()
        set_context(False, None, None, 0, 0,
                    torch.tensor([int(tables[i, 0]) * bs + n for i, n in enumerate(lens)], dtype=torch.int64),
                    torch.tensor([n + 1 for n in lens], dtype=torch.int64), tables,
                    positions=torch.tensor(list(lens), dtype=torch.int64))
        decode = model.compute_logits(model(tok))
        reset_context()
    err_p = float((prefill - torch.from_numpy(z["prefill_logits"])).abs().max())
    err_d = float((decode - torch.from_numpy(z["decode_logits"])).abs().max())
    assert err_p <= 1e-4 and err_d <= 1e-4, (err_p, err_d)
