"""Pairwise human evaluation of model outputs: annotation server, agreement / win-rate metrics, export."""
