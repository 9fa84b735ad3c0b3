"""B200-native weight-placement data plane behind ModelExpress's loader seams.

The compute lives in ``libmxb200.so`` (hand-written sm_100a CUDA behind a C
ABI, see ``include/mxb200.h``); this package is the host-side mirror of the
reference's Python interfaces for the same path:

================================  ===========================================
here                              reference (modelexpress_client/python/modelexpress)
================================  ===========================================
transport.MxbTransport            refit/reshard/transport/base.py Transport
transport.ReadDescriptor          refit/reshard/transport/base.py:26-35
digest.safe_checksum              tensor_utils.py:27-44
digest.tensor_digest              refit/reshard/verify.py:79-155
safetensors_index.parse_safetensors_header   gds_loader.py:245-282
planner.plan_pull_2d              refit/reshard/slice_plan.py:297-339
layout / loader.place_checkpoint  engines/vllm/adapter.py:316-329 (host-staged load)
loader.B200ScatterStrategy        load_strategy/base.py:37-76 LoadStrategy
loader.B200CapturedStrategy       the same plugin, planned from the engine's load_weights
geometry.capture_geometry         refit/reshard/geometry.py:253-309
refit.ReshardReceiver             refit/reshard/receiver.py:336-1043 (data-plane core)
refit.merge_shard_tables          refit/reshard/rendezvous.py:184-272
reshard                           refit/reshard/receiver.py:759-1043 wire + re-slice
installer.MdlLoader               engines/vllm/refit/installer.py:86-191
verify.verify_sources             modelexpress_rl/inference/nixl_staged_transfer.py:529-549
fanout                            nixl_transfer.py:769-952 receive_from_source
engines.vllm.loader.MxModelLoader engines/vllm/loader.py:62-183
engines.sglang.loader.MxModelLoader  engines/sglang/loader.py:44-86
================================  ===========================================

There is no CPU fallback: importing the compute modules without the built
library raises.
"""

__version__ = "0.1.0"
