"""Evaluation library: CI-L0, CI histograms, fresh-PGD recon probes, CE/KL under mask variants."""
