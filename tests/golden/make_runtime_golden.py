"""Generates tests/golden/tiny_llama/: a tiny random-init Llama exported by the REFERENCE'S OWN
exporter, plus the HuggingFace reference outputs the reference validates its runtime against.

Run where the reference tree and `transformers` are present (B200P_REFERENCE_ROOT or argv[1]
names the tree).  Steps, following the reference's Stage-C procedure:
  1. a seeded LlamaForCausalLM (2 layers, hidden 128, 2 query / 1 KV head of dim 64, FFN 256,
     vocab 256; fp16) is saved as a HuggingFace directory;
  2. cdna3-prims/runtime/export_model.py, unmodified, turns it into meta.json + per-tensor .bin
     files (the format cdna3::runtime::ModelLoader reads);
  3. as cdna3-prims/runtime/make_reference.py does (without a tokenizer: the prompt is a seeded
     id sequence), HuggingFace runs the fp16 model on the CPU: ref_logits0.bin = fp32 copy of the
     last prompt token's logits, ref_tokens.txt = prompt + greedy continuation; prompt_ids.txt.
     ref_logits0_f32.bin repeats the first with the weights up-cast to fp32 (no fp16 rounding of
     activations), as a second opinion on where the truth lies.
The HuggingFace working directory is temporary; only the export and the reference outputs are kept.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "tiny_llama")
PROMPT_LEN, MAX_NEW = 40, 12


def main():
    repo = os.path.dirname(os.path.dirname(HERE))
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("B200P_REFERENCE_ROOT", os.path.join(os.path.dirname(repo), "reference"))
    exporter = os.path.join(root, "cdna3-prims", "runtime", "export_model.py")
    if not os.path.exists(exporter):
        raise SystemExit("reference tree not found: pass its root as argv[1] or in B200P_REFERENCE_ROOT")
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0xB205)
    cfg = LlamaConfig(vocab_size=256, hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                      num_key_value_heads=1, max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=10000.0,
                      tie_word_embeddings=False, attention_bias=False, initializer_range=0.08)
    model = LlamaForCausalLM(cfg).half().eval()
    with torch.no_grad():                                   # norm weights away from 1 so that they matter
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_((1.0 + 0.1 * torch.randn(p.shape)).half())
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        hf_dir = os.path.join(tmp, "hf")
        model.save_pretrained(hf_dir, safe_serialization=True)
        subprocess.run([sys.executable, exporter, "--model", hf_dir, "--out", OUT], check=True)
    # meta.json records the temporary path as model_id: replace it with a stable description
    import json
    meta_path = os.path.join(OUT, "meta.json")
    meta = json.load(open(meta_path))
    meta["model_id"] = "random-init LlamaForCausalLM (seed 0xB205), see make_runtime_golden.py"
    json.dump(meta, open(meta_path, "w"), indent=2)

    ids = torch.from_numpy(np.random.default_rng(0xB205).integers(0, cfg.vocab_size, (1, PROMPT_LEN))).long()
    with torch.no_grad():
        logits16 = model(ids).logits[0, -1].float()
        out = model.generate(ids, max_new_tokens=MAX_NEW, do_sample=False, num_beams=1, temperature=None, top_p=None, top_k=None,
                             pad_token_id=0)
        logits32 = model.float()(ids).logits[0, -1].float()
    logits16.numpy().tofile(os.path.join(OUT, "ref_logits0.bin"))
    logits32.numpy().tofile(os.path.join(OUT, "ref_logits0_f32.bin"))
    with open(os.path.join(OUT, "prompt_ids.txt"), "w") as f:
        f.writelines(f"{t}\n" for t in ids[0].tolist())
    with open(os.path.join(OUT, "ref_tokens.txt"), "w") as f:
        f.writelines(f"{t}\n" for t in out[0].tolist())
    srt = np.sort(logits16.numpy())
    print(f"logits std {logits16.std():.3f}, top-2 margin {srt[-1] - srt[-2]:.3f}, "
          f"fp16-vs-fp32 max diff {(logits16 - logits32).abs().max():.4f}; generated {out[0, PROMPT_LEN:].tolist()}")


if __name__ == "__main__":
    main()
