"""cute_triadic_gdn_b200: hand-written sm_100a CUDA kernels for Triadic Gated DeltaNet behind the reference's Python API.

    chunk_gdn_joint       Triadic GDN with autograd, as a plain autograd call
    gdn_joint_call        the same behind torch.library custom ops (one node under torch.compile)
    conv_split_act_call   causal depthwise convolution (width 4) with SiLU on the leading channels only

Same names, signatures, shapes and dtypes as cute_triadic_gdn/__init__.py:7-11 of the reference.

Beyond the reference's surface:

    conv_split_norm_call            the convolution with the layer glue fused in: x -> (q, k, v, k2, q2) as the core
                                    takes them (SiLU / softplus, l2 norms), differentiable
    gdn_joint_decode                one token per sequence on a resident state (continues what
                                    chunk_gdn_joint(..., output_final_state=True) hands out)
    chunk_gdn_joint_segment         one segment of longer sequences: state in / state out, differentiable through both
    context_parallel_joint          sequences split along the token axis over the ranks of a process group (states and
                                    their gradients travel point to point, head groups as a wavefront)
    HostPipeline / gdn_joint_host   inputs and results in pinned host memory; uploads, kernels and downloads of
                                    successive batch slices overlap on three streams (host_pipeline.py)
"""
from .conv_split_act import conv_split_act_call, conv_split_norm_call
from .context_parallel import context_parallel_joint
from .gdn_joint import chunk_gdn_joint, chunk_gdn_joint_segment, gdn_joint_decode
from .host_pipeline import HostPipeline, gdn_joint_host
from .joint_torch_ops import gdn_joint_call

__all__ = ["chunk_gdn_joint", "gdn_joint_call", "conv_split_act_call", "conv_split_norm_call", "gdn_joint_decode", "chunk_gdn_joint_segment",
           "context_parallel_joint", "HostPipeline",
           "gdn_joint_host"]
__version__ = "0.1.0"
