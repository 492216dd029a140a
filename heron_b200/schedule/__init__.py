"""Knob space of the B200 kernels: contexts, schedule rules and the constraint model."""
