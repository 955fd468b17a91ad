"""Failure paths of the boundary, through the C ABI: every refusal is a status with the code the
reference's driver gives for the same mistake, nothing faults, and the device stays usable.

Reference checks mirrored: executable format / version (runtime/driver/nop_executable_cache.cc:97-105,
runtime/driver/TorqExecutable.cc:663-667), binding validation (runtime/driver/torq_command_buffer.c:488-495,
TorqExecutable.cc:512-531), bounded wait (runtime/torq_hw/src/TorqHw.cpp:172-186), host profiling log
(runtime/torq_hw/src/TorqEventLog.cpp:49,95-100)."""
import csv
import ctypes as C
import struct

import numpy as np
import pytest

from gpu_exec import run_graph_gpu
from oracle_exec import run_graph
from torq_b200 import oplist
from torq_b200.oplist import Graph
from torq_b200.quant import quantize_multipliers
from torq_b200.runtime import MEMORY_HOST_PINNED, Binding, Executable, TorqB200Error

pytestmark = pytest.mark.gpu


def _conv_graph(shape=(2, 12, 12, 32), oc=32):
    rng = np.random.default_rng(5)
    g = Graph()
    w = rng.integers(-127, 128, (oc, 1, 1, shape[3]), dtype=np.int8)
    m, s = quantize_multipliers(rng.uniform(0.5, 1.5, oc) * 40.0 / (np.sqrt(shape[3]) * 74 * 74))
    y = g.conv2d(g.input(shape), w, np.round(rng.normal(0, 500, oc)).astype(np.int32), m, s, input_zp=-3, out_zp=4)
    g.output(y)
    x = rng.integers(-128, 128, shape, dtype=np.int8)
    return g, x


def _status(fn, *a):
    with pytest.raises(TorqB200Error) as e:
        fn(*a)
    return e.value.status_name


def test_blob_validation_statuses(device):
    g, _ = _conv_graph()
    blob = bytearray(g.serialize())
    assert _status(Executable, device, bytes(blob[:40])) == "INVALID_ARGUMENT"        # shorter than its header
    bad_magic = bytearray(blob)
    bad_magic[0] ^= 0xFF
    assert _status(Executable, device, bytes(bad_magic)) == "NOT_FOUND"               # another format
    h = oplist.Header.from_buffer_copy(bytes(blob[:80]))
    newer = bytearray(blob)
    off = oplist.Header.version.offset
    newer[off:off + 4] = struct.pack("<I", h.version + 1)
    assert _status(Executable, device, bytes(newer)) == "UNAVAILABLE"                 # version mismatch
    assert _status(Executable, device, bytes(blob[:len(blob) - 64])) == "INVALID_ARGUMENT"  # truncated
    outside = bytearray(blob)
    off = oplist.Header.ops_offset.offset
    outside[off:off + 8] = struct.pack("<Q", len(blob) + 4096)
    assert _status(Executable, device, bytes(outside)) == "INVALID_ARGUMENT"          # section outside the blob
    Executable(device, bytes(blob)).destroy()                                         # the untouched blob loads


def test_binding_validation_statuses(device):
    g, x = _conv_graph()
    ex = Executable(device, g.serialize())
    lib = device._lib
    d_in, d_out = device.alloc(x.nbytes + 64), device.alloc(ex.outputs_info[0].nbytes + 64)
    pinned = device.alloc(x.nbytes, MEMORY_HOST_PINNED)

    def dispatch(entries):
        arr = (Binding * len(entries))()
        for i, (buf, off, length) in enumerate(entries):
            arr[i].buffer, arr[i].offset, arr[i].length = (buf._h if buf is not None else None), off, length
        st = lib.tb200_dispatch(ex._h, arr, len(entries))
        return lib.tb200_status_string(st).decode()

    assert dispatch([(d_in, 0, 0)]) == "INVALID_ARGUMENT"                              # wrong binding count
    assert dispatch([(None, 0, 0), (d_out, 0, 0)]) == "FAILED_PRECONDITION"            # NULL binding
    assert dispatch([(d_in, 0, 16), (d_out, 0, 0)]) == "OUT_OF_RANGE"                  # bound range shorter than the tensor
    assert dispatch([(d_in, x.nbytes + 128, 0), (d_out, 0, 0)]) == "OUT_OF_RANGE"      # offset beyond the buffer
    assert dispatch([(d_in, 8, 0), (d_out, 0, 0)]) == "INVALID_ARGUMENT"               # misaligned address
    assert dispatch([(pinned, 0, 0), (d_out, 0, 0)]) == "FAILED_PRECONDITION"          # host heap bound to a dispatch
    assert dispatch([(d_in, 0, 0), (d_out, 0, 0)]) == "OK"
    device.wait()
    # an imported pointer that is itself misaligned is refused at dispatch, not faulted on
    imp = device.import_pointer(d_in.pointer + 4, x.nbytes)
    assert dispatch([(imp, 0, 0), (d_out, 0, 0)]) == "INVALID_ARGUMENT"
    imp.free()
    # transfers beyond a buffer, including offsets that would wrap a 64-bit sum
    junk = np.zeros(16, np.uint8)
    st = lib.tb200_buffer_upload(d_in._h, C.c_uint64(2 ** 64 - 8), junk.ctypes.data_as(C.c_void_p), 16)
    assert lib.tb200_status_string(st) == b"OUT_OF_RANGE"
    st = lib.tb200_buffer_download(d_in._h, C.c_uint64(d_in.nbytes - 8), junk.ctypes.data_as(C.c_void_p), 16)
    assert lib.tb200_status_string(st) == b"OUT_OF_RANGE"
    for b in (d_in, d_out, pinned):
        b.free()
    ex.destroy()


def test_host_call_null_pointer_is_failed_precondition(device):
    g, x = _conv_graph()
    ex = Executable(device, g.serialize())
    ins = (C.c_void_p * 1)(None)
    out = np.empty(ex.outputs_info[0].shape, np.int8)
    outs = (C.c_void_p * 1)(out.ctypes.data)
    st = device._lib.tb200_invoke_host(ex._h, ins, outs)
    assert device._lib.tb200_status_string(st) == b"FAILED_PRECONDITION"
    ex.invoke_host([x], [out])  # and the executable still works
    assert (out == run_graph(g, [x])[0]).all()
    ex.destroy()


def test_wait_deadline_then_ok(device):
    """A wait shorter than the work answers DEADLINE_EXCEEDED and cancels nothing; a normal wait then succeeds."""
    g, x = _conv_graph((64, 112, 112, 32), 96)
    ex = Executable(device, g.serialize())
    d_in, d_out = device.alloc(x.nbytes), device.alloc(ex.outputs_info[0].nbytes)
    d_in.upload(x)
    device.wait()
    for _ in range(50):
        ex.dispatch([d_in], [d_out])
    st = device._lib.tb200_wait(device._h, 1)
    assert device._lib.tb200_status_string(st) == b"DEADLINE_EXCEEDED"
    device.wait(60.0)
    got = d_out.download(ex.outputs_info[0].shape, np.int8)
    assert (got == run_graph(g, [x])[0]).all()
    d_in.free()
    d_out.free()
    ex.destroy()


def test_bounded_wait_reports_aborted_and_device_stays_usable(device):
    """A kernel wait that nothing completes gives up after its limit, the host wait answers ABORTED once,
    and the next dispatch on the same device is bit-exact."""
    device.probe_bounded_wait(20)
    with pytest.raises(TorqB200Error) as e:
        device.wait(10.0)
    assert e.value.status_name == "ABORTED" and "code 99" in str(e.value)
    device.wait(10.0)  # reported once
    g, x = _conv_graph()
    assert (run_graph_gpu(device, g, [x])[0] == run_graph(g, [x])[0]).all()


def test_profile_csv_uses_the_reference_event_names(device, tmp_path):
    g, x = _conv_graph()
    path = tmp_path / "host_profile.csv"
    device.set_profile_csv(str(path))
    try:
        ex = Executable(device, g.serialize())
        out = np.empty(ex.outputs_info[0].shape, np.int8)
        ex.invoke_host([x], [out])
        d_in = device.alloc(x.nbytes)
        d_in.upload(x)
        device.wait()
        d_in.free()
        ex.destroy()
    finally:
        device.set_profile_csv(None)
    assert (out == run_graph(g, [x])[0]).all()
    rows = list(csv.DictReader(open(path)))
    assert list(rows[0].keys()) == ["dispatch_name", "invocation_id", "action_id", "timestamp_us", "event"]
    known = {"DISPATCH", "DISPATCH_SYNC_BINDINGS_IN", "DISPATCH_SYNC_BINDINGS_OUT", "DISPATCH_EXECUTE_ACTIONS", "NSS_START",
             "HOST_COPY"}
    open_events, last_t = [], -1
    for r in rows:
        name, kind = r["event"].rsplit("_", 1)      # how the reference's reader splits it
        assert name in known and kind in ("BEGIN", "END"), r
        t = int(r["timestamp_us"])                   # whole microseconds, as the reference's reader parses them
        assert t >= last_t, "rows are in time order"
        last_t = t
        key = (name, int(r["action_id"]))
        if kind == "BEGIN":
            open_events.append(key)
        else:
            assert open_events and open_events[-1] == key, f"unbalanced {r}"
            open_events.pop()
    assert not open_events
    names = [r["event"] for r in rows]
    for want in ("DISPATCH_BEGIN", "DISPATCH_SYNC_BINDINGS_IN_BEGIN", "DISPATCH_EXECUTE_ACTIONS_BEGIN", "NSS_START_BEGIN",
                 "DISPATCH_SYNC_BINDINGS_OUT_END", "DISPATCH_END", "HOST_COPY_BEGIN"):
        assert want in names, want
    ops = [r for r in rows if r["event"] == "NSS_START_BEGIN"]
    assert ops and ops[0]["dispatch_name"] == "gemm_i8_tcgen05" and int(ops[0]["action_id"]) == 0


def test_two_devices_in_one_process(device):
    """Function attributes are per device: the same graphs must run on a second GPU of the same process."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from torq_b200.runtime import Device
    g, x = _conv_graph((2, 16, 16, 64), 128)
    want = run_graph(g, [x])[0]
    assert (run_graph_gpu(device, g, [x])[0] == want).all()
    d1 = Device(1)
    try:
        assert (run_graph_gpu(d1, g, [x])[0] == want).all()
        rng = np.random.default_rng(3)
        gc = Graph()
        w = rng.integers(-127, 128, (32, 3, 3, 32), dtype=np.int8)
        m, s = quantize_multipliers(rng.uniform(0.5, 1.5, 32) * 40.0 / (np.sqrt(288) * 74 * 74))
        gc.output(gc.conv2d(gc.input((1, 20, 20, 32)), w, np.zeros(32, np.int32), m, s, pad=(1, 1, 1, 1), input_zp=2, out_zp=-1))
        xc = rng.integers(-128, 128, (1, 20, 20, 32), dtype=np.int8)
        assert (run_graph_gpu(d1, gc, [xc])[0] == run_graph(gc, [xc])[0]).all()
    finally:
        d1.close()
