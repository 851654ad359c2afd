"""Out-of-band infrastructure with the API shape of the reference's helper packages: remote execution
and code push (``bifrost``), GPU inventory / provisioning queries (``broker``), trigram code search
(``csearch``). Everything that would touch a network or a cloud API goes through an injectable
transport, so the logic is exercised offline."""
