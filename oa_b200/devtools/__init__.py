"""Developer tooling of the framework: source gates (package dependency direction, generated tables, kernel audit) and
diagnostics (evidence bundles, replay determinism).  Nothing here is imported by the runtime."""
