"""Make the 1024 location strings ``<loc0000>`` .. ``<loc1023>`` single tokens, idempotently.

Two situations (reference ``src/opentau/datasets/grounding/tokenizer_utils.py:60-140``): a PaliGemma vocabulary already
holds the strings at ids 256000 .. 257023, and registering them only switches the tokenizer to single-token matching (no
new id, no resize); any other vocabulary gets 1024 new ids appended, and the model's input embedding (and its tied
output head, which reads the same parameter here) must grow by as many rows.  The new rows are drawn under a fixed seed
inside a forked RNG, so they are identical across runs and the caller's random stream is untouched.
"""

from __future__ import annotations

import logging

import torch
from torch import nn

LOC_TOKENS: tuple[str, ...] = tuple(f"<loc{i:04d}>" for i in range(1024))
_LOC_EMBEDDING_INIT_SEED = 0x10CC0DE
log = logging.getLogger(__name__)


def resize_embedding(emb: nn.Embedding, new_len: int, std: float = 0.02) -> None:
    """Grows ``emb`` in place to ``new_len`` rows: old rows kept, new rows ~ N(0, std) under the fixed seed."""
    old = emb.weight.data
    if new_len <= old.shape[0]:
        return
    devices = [old.device] if old.is_cuda else []
    with torch.random.fork_rng(devices=devices):
        torch.manual_seed(_LOC_EMBEDDING_INIT_SEED)
        extra = torch.empty(new_len - old.shape[0], old.shape[1], dtype=torch.float32).normal_(0.0, std)
    emb.weight = nn.Parameter(torch.cat([old, extra.to(old.device, old.dtype)], 0), requires_grad=emb.weight.requires_grad)
    emb.num_embeddings = new_len


def _input_embedding(model) -> nn.Embedding | None:
    if hasattr(model, "get_input_embeddings"):
        return model.get_input_embeddings()
    for name, mod in model.named_modules():
        if name.endswith("embed_tokens") and isinstance(mod, nn.Embedding):
            return mod
    return None


def ensure_loc_tokens(tokenizer, model=None) -> int:
    """Returns the number of NEW ids (0 for a PaliGemma vocabulary and for every later call)."""
    before = len(tokenizer)
    try:
        from transformers.tokenization_utils_base import AddedToken, PreTrainedTokenizerBase
        is_hf = isinstance(tokenizer, PreTrainedTokenizerBase)
    except ImportError:  # pragma: no cover
        is_hf = False
    if is_hf:
        tokenizer.add_tokens([AddedToken(t, special=True, normalized=False) for t in LOC_TOKENS], special_tokens=True)
    else:
        tokenizer.add_tokens(list(LOC_TOKENS), special_tokens=True)
    n_new = len(tokenizer) - before
    if n_new > 0 and model is not None:
        if hasattr(model, "resize_token_embeddings"):
            devices = [d for d in range(torch.cuda.device_count())] if torch.cuda.is_available() else []
            with torch.random.fork_rng(devices=devices):
                torch.manual_seed(_LOC_EMBEDDING_INIT_SEED)
                model.resize_token_embeddings(len(tokenizer))
        else:
            emb = _input_embedding(model)
            if emb is None:
                raise ValueError("the model exposes no input embedding to resize")
            resize_embedding(emb, len(tokenizer))
        log.info("appended %d location tokens; embedding table resized to %d rows", n_new, len(tokenizer))
    return n_new
