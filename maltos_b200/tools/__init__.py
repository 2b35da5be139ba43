"""Command-line tools: training entry, synthetic benchmark harness, checkpoint conversion, data preparation."""
