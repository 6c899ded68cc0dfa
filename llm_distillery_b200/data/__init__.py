"""Data plane: JSONL reading, tokenisation with content ranges, vocab families, SHA sync, chunk planning, HDF5 store."""
