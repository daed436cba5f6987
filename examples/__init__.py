"""Example graphs (reference: ``examples/``)."""
