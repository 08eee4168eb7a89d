"""The inventory's workload table builds valid arguments for every registered kernel name it lists (no GPU)."""

from nano_omni_b200 import inventory, kernels, tune


def test_every_listed_workload_constructs():
    registry = kernels.classes()
    listed = set()
    for name, fields, _ in inventory.workloads(4096, 4):
        cls = registry[name]
        workload = tune.workload_of(cls, fields)
        arguments = cls.make_arguments(workload)
        assert cls.make_workload(arguments) == workload, name  # the reference's round-trip invariant
        assert inventory.argument_bytes(arguments) > 0
        listed.add(name)
    # everything on the attention path is in the table (helpers without a tuning shape aside)
    missing = set(registry) - listed - {"sol_nvfp4_pool", "hadamard128_heads"}
    assert not missing, missing
