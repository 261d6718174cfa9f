"""Selection plugins: ``topk`` with its histogram / exact / adaptive methods."""
