"""Host logic of the generic QEP driver that needs no GPU: capturing layer inputs chunk by chunk."""

import torch

from onecompression_b200.qep import capture_input_activations


def test_capture_in_chunks_equals_one_pass_and_honours_exclusions():
    torch.manual_seed(0)

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(50, 16)
            self.a = torch.nn.Linear(16, 24)
            self.mlp = torch.nn.ModuleDict({"down_proj": torch.nn.Linear(24, 16)})
            self.calls = 0

        def forward(self, input_ids, use_cache=False):
            self.calls += 1
            h = torch.relu(self.a(self.emb(input_ids)))
            return self.mlp["down_proj"](h)

    net = Net()
    ids = torch.randint(0, 50, (10, 7))
    names = {net.a: "a", net.mlp["down_proj"]: "mlp.down_proj"}
    whole = capture_input_activations(net, {"input_ids": ids}, names, batch_size=10)
    parts = capture_input_activations(net, {"input_ids": ids, "use_cache": False}, names, batch_size=4)
    assert set(whole) == {"a", "mlp.down_proj"}
    assert whole["a"].shape == (10, 7, 16) and whole["mlp.down_proj"].shape == (10, 7, 24)
    for k in whole:
        assert torch.equal(whole[k], parts[k])
    only = capture_input_activations(net, {"input_ids": ids}, names, exclude_layer_keywords=["mlp.down_proj"])
    assert set(only) == {"a"}
    # a pass for one early layer stops there
    seen = []
    handle = net.mlp["down_proj"].register_forward_hook(lambda *_: seen.append(1))
    capture_input_activations(net, {"input_ids": ids}, {net.a: "a"}, batch_size=5, stop_after_last=True)
    handle.remove()
    assert not seen
