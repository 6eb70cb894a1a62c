"""Optimizer-state checkpoints in Volta's StateDict container (bincode 2, standard config)."""
import os
import struct

import numpy as np
import pytest


def test_bincode_varint_and_layout_known_answers():
    """The published bincode `standard()` integer encoding and the field order of
    BTreeMap<String, TensorData { data, shape }> (src/io.rs:15-22)."""
    from volta_b200.checkpoint import _put_varint, decode_state_dict, encode_state_dict
    for v, expect in ((0, b"\x00"), (250, b"\xfa"), (251, b"\xfb\xfb\x00"), (65535, b"\xfb\xff\xff"),
                      (65536, b"\xfc\x00\x00\x01\x00"), (1 << 32, b"\xfd" + struct.pack("<Q", 1 << 32))):
        out = bytearray()
        _put_varint(out, v)
        assert bytes(out) == expect
    blob = encode_state_dict({"b": (np.array([1.5, -2.0], np.float32), (2,)), "a": (np.array([0.25], np.float32), (1, 1))})
    expect = (b"\x02"                                                    # two entries, in key order
              b"\x01a" b"\x01" + struct.pack("<f", 0.25) + b"\x02\x01\x01"   # "a": data [0.25], shape [1, 1]
              b"\x01b" b"\x02" + struct.pack("<ff", 1.5, -2.0) + b"\x01\x02")
    assert blob == expect
    back = decode_state_dict(blob)
    assert list(back) == ["a", "b"] and back["b"][1] == (2,) and np.array_equal(back["b"][0], [1.5, -2.0])


def test_large_tensor_round_trip():
    from volta_b200.checkpoint import decode_state_dict, encode_state_dict
    rng = np.random.default_rng(0)
    state = {f"optimizer.state0.{i}": (rng.standard_normal(n).astype(np.float32), (n,)) for i, n in enumerate((1, 300, 70000))}
    back = decode_state_dict(encode_state_dict(state))
    for k, (d, s) in state.items():
        assert back[k][1] == s and np.array_equal(back[k][0].view(np.uint32), d.view(np.uint32))


def test_safetensors_layout_known_answer_and_library_reads_it(tmp_path):
    """The published SafeTensors layout, byte for byte, and a cross-check with the safetensors
    package (the Python binding of the crate Volta links, src/io.rs:6)."""
    from volta_b200.checkpoint import decode_safetensors, encode_safetensors
    state = {"b": (np.array([1.5, -2.0], np.float32), (2,)), "a": (np.array([0.25], np.float32), (1, 1))}
    blob = encode_safetensors(state)
    header = b'{"a":{"dtype":"F32","shape":[1,1],"data_offsets":[0,4]},"b":{"dtype":"F32","shape":[2],"data_offsets":[4,12]}}'
    header += b" " * (-len(header) % 8)
    assert blob == struct.pack("<Q", len(header)) + header + struct.pack("<fff", 0.25, 1.5, -2.0)
    back = decode_safetensors(blob)
    assert list(back) == ["a", "b"] and back["a"][1] == (1, 1) and np.array_equal(back["b"][0], [1.5, -2.0])
    st = pytest.importorskip("safetensors.numpy")
    path = os.path.join(tmp_path, "s.safetensors")
    with open(path, "wb") as fh:
        fh.write(blob)
    lib = st.load_file(path)
    assert lib["a"].shape == (1, 1) and np.array_equal(lib["b"], [1.5, -2.0])
    theirs = st.save({"optimizer.t": np.array([7.0], np.float32), "optimizer.state0.0": np.arange(6, dtype=np.float32).reshape(2, 3)})
    mine = decode_safetensors(theirs)
    assert mine["optimizer.state0.0"][1] == (2, 3) and mine["optimizer.t"][0][0] == 7.0
    with pytest.raises(ValueError):
        decode_safetensors(blob[:20])


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["opt.bin", "opt.safetensors"])
def test_resume_from_checkpoint_is_bit_identical(engine, tmp_path, name):
    from volta_b200 import Adam, Tensor
    from volta_b200.checkpoint import load_optimizer_state, save_optimizer_state
    rng = np.random.default_rng(3)
    shapes = [(40, 25), (7,), (1000,)]
    p0 = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    grads = [[(rng.standard_normal(s) * 0.01).astype(np.float32) for s in shapes] for _ in range(5)]
    a = [Tensor(p.copy()) for p in p0]
    opt_a = Adam(a, 1e-3, (0.9, 0.999), 1e-8, 0.01, engine=engine)
    for g in grads[:3]:
        for t, gi in zip(a, g):
            t.grad = gi
        opt_a.step()
    path = os.path.join(tmp_path, name)
    save_optimizer_state(opt_a, path)
    b = [Tensor(t.data.copy()) for t in a]
    opt_b = Adam(b, 1e-3, (0.9, 0.999), 1e-8, 0.01, engine=engine)
    load_optimizer_state(opt_b, path)
    assert opt_b.t == 3
    for g in grads[3:]:
        for ta, tb, gi in zip(a, b, g):
            ta.grad = gi
            tb.grad = gi
        opt_a.step()
        opt_b.step()
    for ta, tb in zip(a, b):
        assert np.array_equal(ta.data.view(np.uint32), tb.data.view(np.uint32))
    opt_a.close()
    opt_b.close()
