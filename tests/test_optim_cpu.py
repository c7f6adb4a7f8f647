

def test_master_weights_follow_parameters_overwritten_without_the_optimizer():
    """bf16 parameters owned by a fused optimizer are overwritten from outside (what a broadcast or a loaded state
    dict does): the fp32 master copy must follow, or the next step writes the stale values back."""
    import torch
    from tips_b200.ops.optim import FusedSGD, refresh_masters_of
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 4).to(torch.bfloat16)
    opt = FusedSGD(lin.parameters(), lr=0.0)   # lr 0: a step only writes the master copy back
    opt.build()
    new_w = torch.full_like(lin.weight, 0.5)
    with torch.no_grad():
        lin.weight.copy_(new_w)
    assert refresh_masters_of(lin.state_dict().values()) == 1
    lin(torch.ones(2, 8, dtype=torch.bfloat16)).sum().backward()
    opt.step()
    assert torch.equal(lin.weight.detach(), new_w)
