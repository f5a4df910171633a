"""Experiment harness: offline / online / ablation runs, summaries, published comparison numbers."""
