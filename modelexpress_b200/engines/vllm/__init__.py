"""vLLM integration: ``MxModelLoader`` with the reference's three entry points."""
