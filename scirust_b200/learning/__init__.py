"""Classical learning algorithms on tensors (float64 by default, any device): regression (kernel ridge, robust,
high-breakdown, isotonic, quantile, influence diagnostics), Gaussian processes, unsupervised learning and anomaly
detection, forecasting, and policy-gradient reinforcement learning. Every fit is a handful of batched linear-algebra
calls, so candidate subsets, restarts and query batches are evaluated together rather than in host loops.
Reference counterpart: scirust-learning, scirust-gp, scirust-unsupervised, scirust-forecast and scirust-rl-algo."""
from .regression import (IsotonicRegression, KernelRidgeRegression, LinearModel, fit_high_breakdown,  # noqa: F401
                         fit_multi_output_robust, fit_quantile_regression, fit_robust_regression, influence_report)
from .gp import GaussianProcess, Matern32, Matern52, Rbf  # noqa: F401
