"""Evaluation: bits-per-byte over scored spans, batched greedy generation on caches, long-context position buckets,
synthetic recall probes, multiple choice, GDN state diagnostics, resumable scoring units."""
