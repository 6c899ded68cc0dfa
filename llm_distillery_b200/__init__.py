"""B200-native offline LLM distillation framework (collect teacher top-K log-probs -> HDF5 -> train student).

Sub-packages: ``config``/``cli`` (config.json + flags, orchestration), ``data`` (JSONL, tokenisation, SHA sync,
HDF5 store), ``models`` (Llama-family graph on the sm_100a kernels), ``ops`` (kernel bindings + CPU oracles),
``loss``, ``engine`` (single / DDP / FSDP training), ``parallel`` (NVLink P2P collectives, TP), ``collect``,
``ckpt``, ``obs``, ``align`` (cross-tokenizer trie), ``utils`` (offline dataset tools).
"""
__version__ = "0.1.0"
