"""Offline tools: checkpoint conversion, sample packing, dataset format converters, parquet to JSONL, and the
synthetic fixtures (tokenizer / model folders / datasets) used by tests and benchmarks."""
