# SPDX-License-Identifier: Apache-2.0
"""Reporting stack: orchestrator hook, scalar extraction, Rich / TensorBoard / JSON-lines reporters."""
from nvalchemi_toolkit_b200.hooks.reporting._core import (DEFAULT_REPORT_STAGES, Reporter, ReporterMessage,
                                                         ReportingErrorPolicy, ReportingOrchestrator, ReportingState,
                                                         ScalarSnapshot, collect_scalars, extract_dynamics_scalars,
                                                         extract_loss_scalars, extract_optimizer_lr_scalars,
                                                         extract_progress_scalars, extract_scalars, reduce_scalars_across_ranks)
from nvalchemi_toolkit_b200.hooks.reporting._core import ScalarCallback
from nvalchemi_toolkit_b200.hooks.reporting._layouts import (BaseDashboardLayout, CompactLayout, DynamicsLayout,
                                                            TrainingLayout, resolve_layout, text_plot)
from nvalchemi_toolkit_b200.hooks.reporting._reporters import (JSONLReporter, RichLayout, RichReporter,
                                                              TensorBoardReporter, TensorBoardWriter, sparkline)

__all__ = ["DEFAULT_REPORT_STAGES", "Reporter", "ReporterMessage", "ReportingErrorPolicy", "ReportingOrchestrator",
           "ReportingState", "ScalarSnapshot", "collect_scalars", "extract_dynamics_scalars", "extract_loss_scalars",
           "extract_optimizer_lr_scalars", "extract_progress_scalars", "reduce_scalars_across_ranks", "JSONLReporter",
           "RichLayout", "RichReporter", "TensorBoardReporter", "sparkline", "BaseDashboardLayout", "CompactLayout",
           "DynamicsLayout", "TrainingLayout", "resolve_layout", "text_plot", "extract_scalars", "ScalarCallback",
           "TensorBoardWriter"]

#: the layout classes under the names the reference exports them
BaseRichLayout, TrainingRichLayout, DynamicsRichLayout = BaseDashboardLayout, TrainingLayout, DynamicsLayout
__all__ += ["BaseRichLayout", "TrainingRichLayout", "DynamicsRichLayout"]
