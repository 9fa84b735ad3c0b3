"""Import-path shim: lets vLLM find ``modelexpress.engines.vllm.loader`` (add ``modelexpress_b200/shim`` to PYTHONPATH)."""
