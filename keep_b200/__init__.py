"""keep_b200: the routed E8P expert path of jackmaxwil/keep on NVIDIA B200 (sm_100a).

Modules, by the reference interface they stand in for:

``vq``               codebooks and ``decode_weight_matrix`` (``keep.vq.e8``)
``kernels``          ``vq_qmv``, ``vq_qmm``, the few-token ``e8p_m1`` / ``e8_1bit_m1`` / ``e8p_nested_m1`` operators
``vq_switch``        ``gather_vqmm``, ``gather_vqmm_sorted_routes``, ``vq_switch_qmv``
``prefill``          the sorted-route grouped product on the tensor-core kernels
``switch``           ``QuantizedVQSwitchLinear``, ``QuantizedVQSwitchGLU``
``router``           served / demand top-k with residency bias and admission flags
``moe``              one routed MoE layer call (router, experts, combine) without a host round trip
``residency``        admission / eviction policy on the device and the slot installer
``expert_parallel``  experts sharded over the GPUs of a node (peer-memory or NCCL exchange)
``io``               ``layer-NN.npz`` files and safetensors switch projections
``torch_ops``        the same operators registered as PyTorch custom ops (``torch.ops.keepvq.*``); importing it registers them

Everything computes on the GPU through ``libkeepvq.so`` (``include/keepvq.h``); build it with
``python -m keep_b200.build``.  There is no CPU path.
"""
