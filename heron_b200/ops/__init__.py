"""Operator definitions on the hot path, under the reference's names and signatures."""
