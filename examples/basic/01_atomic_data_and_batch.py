# SPDX-License-Identifier: Apache-2.0
"""AtomicData, Batch, indexing and round trips."""
import torch

from nvalchemi_toolkit_b200 import AtomicData, Batch

water = AtomicData(atomic_numbers=torch.tensor([8, 1, 1]),
                   positions=torch.tensor([[0.0, 0.0, 0.0], [0.96, 0.0, 0.0], [-0.24, 0.93, 0.0]]))
co2 = AtomicData(atomic_numbers=torch.tensor([6, 8, 8]),
                 positions=torch.tensor([[0.0, 0.0, 0.0], [1.16, 0.0, 0.0], [-1.16, 0.0, 0.0]]))
methane = AtomicData(atomic_numbers=torch.tensor([6, 1, 1, 1, 1]), positions=torch.randn(5, 3))
batch = Batch.from_data_list([water, co2, methane])
print(batch)
print("atoms per system:", batch.num_nodes_list, "| batch_ptr:", batch.batch_ptr.tolist())
print("masses were filled from the periodic table:", batch.atomic_masses[:3].tolist())
sub = batch.index_select([0, 2])                    # a new batch with systems 0 and 2
print("selected:", sub.num_graphs, "systems,", sub.num_nodes, "atoms")
batch.add_key("label", torch.tensor([[1.0], [2.0], [3.0]]), level="system")
again = batch.get_data(1)                           # back to a single AtomicData
print("system 1 label:", float(batch.label[1]), "| atoms:", again.atomic_numbers.tolist())
