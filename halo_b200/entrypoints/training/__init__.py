"""One ``main()`` per training method; ``halo_b200 launch <method> <config>`` runs them."""
