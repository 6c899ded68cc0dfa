"""Vocabulary families. A family is identified by the SHA-256 of the sorted base vocabulary (all tokens minus
added tokens); models of one family share token ids, so their distributions can be mixed directly
(reference: utils/vocab_utils.py). Hashes and per-family BOS ids are facts about public tokenizers."""
from __future__ import annotations

import hashlib

# sha256(sorted base vocab joined) -> family name
SHA_TO_FAMILY = {
    "154a07d332d0466ce54d5e83190930dc872c95777c493653c48d6b6b01891377": "mistral",
    "88dfafd1e6cd6fc3cf71600f1c8590ec6b457263267d801636320000a6f687e3": "llama_1|2",
    "7f1739ca602e925d6c93e42c0d4d4f6f607169f5b016d5d322e4ec42a1c7c563": "llama_3",
    "748d7e81288e3b759c4458794fee17f546a07e08e70832d2f04486cd1fc76121": "command-r",
    "12c2a843415f76681408ba2645bb7ea68fc00e864afbfa408193159f847fbe4b": "dbrx",
    "f41d538d54aa627ad2d1a7d853759ac104b94775a5de51e6e6e6e112fb32c1de": "gpt2",
    "e59f183b9781a484efd580deda830bd952f7d3694c4648d41d295284a48f2945": "codeqwen",
    "5520ff09e574cbb231f2baf283bd1a2e358b5d747c1a6aaa6402ee03991a409d": "qwen_1.5",
    "347b0481e0536ab58d630b461c8bbb9dceb8b1a3ff6b9250c73bcd423e64fa71": "gptneox",
    "9eb38d83274ea4aac4d1a037331c7b9f51ee5a74bc2ff9d85f3c1b7a944f2fd0": "gemma",
    "b6f82ad160f599b1dd5bec8987acb5a316423d04de3123fa1eb0c8f1ba7f5568": "gemma",
    "f6556674148d92703237bab474c2cf220255926e7b6811e526b072d0ed086beb": "yi",
    "2e7d13c6f9a9825b1dfeb645fe3130b118e4c119bdf0460be06bd7e2d7660728": "deepseek",
    "62947c306f3a11187ba2a4a6ea25de91ce30c5724e6b647a1d6f0f8868217ead": "deepseek_1.5",
    "94c18f1464d6aeb4542dff2fb8dc837e131e39853d86707eea683470c7344480": "T5",
    "cabd41803ba4aa362c59603aa9fedd80d8eab202708beccce9f4e1e0b58eaf3f": "codellama",
    "c2ed819dc3c535a3a64a10d492a39baa87b9cc7aa0a2c72adecc1b31e3e1b544": "jamba",
}

# None = ask the tokenizer
FAMILY_BOS_ID = {
    "mistral": 1, "llama_1|2": 1, "llama_3": 128000, "command-r": 5, "dbrx": None, "gpt2": 50256, "codeqwen": 1,
    "qwen_1.5": None, "gptneox": 50256, "gemma": 2, "yi": 1, "deepseek": None, "deepseek_1.5": 100000, "T5": None,
    "codellama": 1, "jamba": 1,
}


def try_load_tokenizer(model_path: str):
    from transformers import AutoTokenizer
    try:
        return AutoTokenizer.from_pretrained(model_path, legacy=False)
    except Exception as e:  # noqa: BLE001 - any loader failure means "no tokenizer here"
        raise ValueError(f"Tokenizer for {model_path} could not be loaded") from e


def get_tokenizer_sha(tokenizer=None, model_path: str = "") -> str:
    tokenizer = try_load_tokenizer(model_path) if tokenizer is None else tokenizer
    base = sorted(set(tokenizer.get_vocab().keys()) - set(tokenizer.get_added_vocab().keys()))
    return hashlib.sha256("".join(base).encode()).hexdigest()


def get_vocab_family(tokenizer=None, model_path: str = "") -> str:
    """Known family name, or ``"Unknown"``. Two unknown tokenizers are still told apart: callers that need that
    use :func:`vocab_identity`."""
    return SHA_TO_FAMILY.get(get_tokenizer_sha(tokenizer, model_path), "Unknown")


def vocab_identity(tokenizer=None, model_path: str = "") -> str:
    """Family name when known, else ``"sha:<first 16 hex>"`` - so that two different unregistered vocabularies
    never compare equal (the reference lumps every unregistered tokenizer into "Unknown")."""
    sha = get_tokenizer_sha(tokenizer, model_path)
    return SHA_TO_FAMILY.get(sha, f"sha:{sha[:16]}")


def get_family_bos_id(vocab_family: str, tokenizer=None, model_path: str = ""):
    bos = FAMILY_BOS_ID.get(vocab_family)
    if bos is None:
        tokenizer = try_load_tokenizer(model_path) if tokenizer is None else tokenizer
        bos = tokenizer.bos_token_id
    return bos
