"""Cross-cutting helpers: tracing (:mod:`astrai_b200.utils.trace`)."""
