"""``modelexpress.engines.vllm.loader`` as vLLM imports it, backed by the B200 path."""

from modelexpress_b200.engines.vllm.loader import MxModelLoader  # noqa: F401
