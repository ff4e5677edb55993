"""A parameter server for one box of NVLink-connected B200 GPUs, with the public API, configuration files and
model output of dmlc/parameter_server.

Sub-packages (nothing heavy is imported here; import what you use):

``system``     the C++ host runtime (``system.core``: nodes, customers, executors with timestamps and ``wait_time``,
               KVVector / KVMap / KVLayer, filters, readers, utilities), in-process clusters, job control, launchers
``app``        the linear-method application on GPUs (``python -m parameter_server_b200.app.linear -app_file x.conf``)
               and its node layer (scheduler / server / worker roles of every rank)
``models``     sparse logistic regression with FTRL / AdaGrad / SGD (``sparse_lr``) and Darlin block coordinate
               descent (``darlin``, ``darlin_prep``) on the device data plane
``parallel``   the device data plane: symmetric heap over CUDA IPC (``fabric``), fused push / pull / apply kernels
               (``dataplane``), wide values through tensor-core tiles (``wide``), the NCCL comparison arm
``parameter``  device KV containers with the reference's Push / Pull / Wait conventions (``kv``, ``kv_layer``) and as
               customers of the host runtime (``kv_nodes``)
``ops``        thin wrappers over the CUDA library (``localize``, ``filters``), per-kernel probes (``microbench``)
``utils``      CPU oracles, synthetic and text data, binary matrix files, checkpoints, the data tool

``_build`` compiles everything in-tree: ``libpsb_cuda.so`` (nvcc, sm_100a), the ``_core`` module,
``bin/psb_linear`` and the static libraries for C++ programs.
"""

__version__ = "0.2.0"
