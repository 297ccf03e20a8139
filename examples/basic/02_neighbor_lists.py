# SPDX-License-Identifier: Apache-2.0
"""Dense neighbour matrices and COO lists, with periodic images."""
import torch

from nvalchemi_toolkit_b200 import Batch, neighbors
from nvalchemi_toolkit_b200.benchmark import systems
from nvalchemi_toolkit_b200.models.base import NeighborListFormat

batch = Batch.from_data_list([systems.fcc(3, a=4.05, z=13, noise=0.0), systems.bcc_iron(3, noise=0.0)])
neighbors.compute_neighbors(batch, cutoff=3.0)
print("matrix:", tuple(batch.neighbor_matrix.shape), "| neighbours of atom 0:", int(batch.num_neighbors[0]))
print("fcc Al has 12 nearest neighbours:", bool((batch.num_neighbors[:108] == 12).all()))
print("bcc Fe has 8 + 6 within 3.0 A:", bool((batch.num_neighbors[108:] == 14).all()))
neighbors.compute_neighbors(batch, cutoff=3.0, format=NeighborListFormat.COO)
print("COO edges:", tuple(batch.neighbor_list.shape), "| shifts:", tuple(batch.neighbor_list_shifts.shape))
