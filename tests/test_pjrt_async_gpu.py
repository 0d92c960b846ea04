"""PJRT_Buffer_ToHostBuffer returns while the bytes travel: its event is pending until the client's transfer stream has
delivered them, a program may be executed in between, and a buffer may be destroyed with its transfer in flight."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

SCALE = """
module @scale {
  func.func @main(%a: tensor<4194304xf32>, %s: tensor<f32>) -> (tensor<4194304xf32>) {
    %b = stablehlo.broadcast_in_dim %s, dims = [] : (tensor<f32>) -> tensor<4194304xf32>
    %0 = stablehlo.multiply %a, %b : tensor<4194304xf32>
    return %0 : tensor<4194304xf32>
  }
}
"""


def test_transfers_overlap_the_next_execution_and_deliver_the_right_bytes():
    from metalhlo_b200 import pjrt

    host = pjrt.Host()
    exe = host.compile(SCALE)
    x = np.arange(4194304, dtype=np.float32)
    xb = host.buffer(x)
    pinned = [torch.empty(4194304, dtype=torch.float32).pin_memory() for _ in range(2)]
    waits = []
    for step in range(6):
        out = exe.execute([xb, host.buffer(np.float32(step + 1))])[0]
        if len(waits) == 2:  # the transfer that used this pinned buffer two steps ago
            wait, want = waits.pop(0)
            wait()
            np.testing.assert_array_equal(pinned[step % 2].numpy(), want)
        waits.append((out.to_host_pointer_start(pinned[step % 2].data_ptr(), 4 * 4194304), x * np.float32(step + 1)))
        del out  # destroyed with its transfer possibly in flight: destruction waits for that transfer
    for i, (wait, want) in enumerate(waits):
        wait()
        np.testing.assert_array_equal(pinned[(4 + i) % 2].numpy(), want)


def test_the_synchronous_call_still_waits():
    from metalhlo_b200 import pjrt

    host = pjrt.Host()
    exe = host.compile(SCALE)
    x = np.linspace(-1, 1, 4194304, dtype=np.float32)
    out = exe.execute([host.buffer(x), host.buffer(np.float32(3))])[0]
    got = out.to_numpy()
    np.testing.assert_array_equal(got, x * np.float32(3))
