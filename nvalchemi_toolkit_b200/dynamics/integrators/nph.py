# SPDX-License-Identifier: Apache-2.0
"""Isoenthalpic-isobaric (NPH) dynamics: the Martyna-Tobias-Klein barostat of :class:`NPT` without the two Nose-Hoover
chains (reference ``nvalchemi/dynamics/integrators/nph.py`` and the ``nph_*`` ops).  The enthalpy ``E + KE + p V`` plus the
barostat's kinetic energy is conserved; ``temperature`` only sets the barostat mass ``W = (N_f + 3) kT tau_b^2``."""
from __future__ import annotations

from typing import Any

from nvalchemi_toolkit_b200.dynamics.integrators.npt import NPT


class NPH(NPT):
    __dd_thermo_kind__ = "nph"
    _thermostat = False

    def __init__(self, model: Any, dt: float, pressure: float, barostat_time: float,
                 pressure_coupling: str = "isotropic", temperature: float = 300.0, n_steps: int | None = None,
                 hooks: list | None = None, convergence_hook: Any = None, **kwargs: Any) -> None:
        super().__init__(model=model, dt=dt, temperature=temperature, pressure=pressure, barostat_time=barostat_time,
                         thermostat_time=barostat_time, pressure_coupling=pressure_coupling, n_steps=n_steps, hooks=hooks,
                         convergence_hook=convergence_hook, **kwargs)
