"""Write a small Llama-architecture model directory (config + word-level tokenizer, no weights).

There is no network and no checkpoint on the test machines, so the serving drivers run vLLM with
``--load-format dummy`` on a directory made here.  The shape keeps what matters for decode context
parallelism: grouped-query attention with ONE KV head (so that tensor parallel ranks replicate KV and
DCP can shard the sequence instead) and head_dim 128.

    python -m benchmarks.serving.tiny_model OUT_DIR [--layers 4] [--hidden 1024] [--heads 8] [--vocab 2048]
"""
from __future__ import annotations

import argparse
import json
import os


def write_tiny_model(out_dir: str, *, layers: int = 4, hidden: int = 1024, heads: int = 8, kv_heads: int = 1,
                     vocab: int = 2048, max_len: int = 131072) -> str:
    os.makedirs(out_dir, exist_ok=True)
    assert hidden % heads == 0
    cfg = {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama",
        "hidden_size": hidden, "intermediate_size": hidden * 2, "num_hidden_layers": layers,
        "num_attention_heads": heads, "num_key_value_heads": kv_heads, "head_dim": hidden // heads,
        "vocab_size": vocab, "max_position_embeddings": max_len, "rms_norm_eps": 1e-5,
        "rope_theta": 500000.0, "hidden_act": "silu", "tie_word_embeddings": False,
        "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0,
        "attention_bias": False, "mlp_bias": False,
    }
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    with open(os.path.join(out_dir, "generation_config.json"), "w") as f:
        json.dump({"bos_token_id": 1, "eos_token_id": 2, "pad_token_id": 0}, f)

    from tokenizers import Tokenizer, models, pre_tokenizers
    words = ["<pad>", "<s>", "</s>", "<unk>"] + [_word(i) for i in range(vocab - 4)]
    tok = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    # no decoder: transformers joins word-level tokens with single spaces, which round-trips the prompts above
    tok.save(os.path.join(out_dir, "tokenizer.json"))
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"tokenizer_class": "PreTrainedTokenizerFast", "bos_token": "<s>", "eos_token": "</s>",
                   "unk_token": "<unk>", "pad_token": "<pad>", "model_max_length": max_len,
                   "clean_up_tokenization_spaces": False}, f)
    with open(os.path.join(out_dir, "special_tokens_map.json"), "w") as f:
        json.dump({"bos_token": "<s>", "eos_token": "</s>", "unk_token": "<unk>", "pad_token": "<pad>"}, f)
    return out_dir


def _word(i: int) -> str:
    """Vocabulary word i: at most four characters with its separating space for vocabularies up to 4096
    (servers bound the prompt's character count by a few characters per token of context before tokenising)."""
    return format(i, "03x")


def synthetic_prompt(n_tokens: int, seed: int = 0, vocab: int = 2048) -> str:
    """A deterministic prompt of exactly ``n_tokens`` word-level tokens (plus BOS if the server adds one)."""
    import random
    rng = random.Random(seed)
    return " ".join(_word(rng.randrange(vocab - 4)) for _ in range(n_tokens))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("out_dir")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=1)
    ap.add_argument("--vocab", type=int, default=2048)
    a = ap.parse_args(argv)
    print(write_tiny_model(a.out_dir, layers=a.layers, hidden=a.hidden, heads=a.heads, kv_heads=a.kv_heads, vocab=a.vocab))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
