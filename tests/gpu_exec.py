"""Runs a Graph on the GPU through the C ABI (executable create -> dispatch -> download)."""
import numpy as np

from torq_b200.runtime import Executable


def run_graph_gpu(device, graph, inputs, host_call=False):
    ex = Executable(device, graph.serialize())
    try:
        if host_call:
            outs = [np.empty(o.shape, o.np_dtype) for o in ex.outputs_info]
            ex.invoke_host([np.ascontiguousarray(a) for a in inputs], outs)
            return outs
        ins = [device.alloc(i.nbytes) for i in ex.inputs_info]
        outs = [device.alloc(o.nbytes) for o in ex.outputs_info]
        for b, a in zip(ins, inputs):
            b.upload(np.ascontiguousarray(a))
        ex.dispatch(ins, outs)
        res = [b.download(o.shape, o.np_dtype) for b, o in zip(outs, ex.outputs_info)]
        for b in ins + outs:
            b.free()
        return res
    finally:
        ex.destroy()
