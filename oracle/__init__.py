"""CPU oracle of the low-precision linear path.  Test infrastructure only: the shipped
package never imports it; only tests/, the smoke check and the bench's CPU-baseline
leg do, and only as the checker."""
