"""SGLang integration: ``MxModelLoader`` with the reference's signature."""
