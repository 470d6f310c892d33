"""Multi-GPU plumbing: rank bootstrap over ``torch.distributed``, host collective injection for the
CPU learners, and the symmetric-heap handle exchange for the in-kernel NVLink collectives."""
